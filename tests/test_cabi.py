"""The C-ABI library builds for sm_100a without a GPU, loads, and exports every
function that include/attn_b200.h declares.  No compute call is made here."""

import ctypes
import os
import re

from core.native import lib

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "attn_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(attn_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_functions_all_exported(native_lib):
    names = declared_functions()
    assert "attn_b200_parallel_fwd" in names and "attn_b200_mla_decode" in names and "attn_b200_linear_fwd" in names
    dll = ctypes.CDLL(lib.LIB_PATH)
    for n in names:
        assert hasattr(dll, n), f"{n} declared in attn_b200.h but not exported"


def test_binding_covers_header():
    assert set(declared_functions()) <= set(lib.SIGNATURES), "ctypes binding misses a declared entry point"


def test_struct_layouts_match_header(tmp_path):
    """sizeof / offsetof of every argument struct as the C compiler sees the header, against the ctypes mirrors"""
    import subprocess
    probes = {
        "AttnB200ParallelArgs": (lib.ParallelArgs, ["o", "seq_kv", "o_stride", "heads_kv", "fparams", "custom_stride", "mask_left", "mask_right", "num_splits", "workspace", "workspace_bytes"]),
        "AttnB200LinearArgs": (lib.LinearArgs, ["log_decay", "dim_v", "normalize", "q_scale", "workspace", "workspace_bytes", "precise", "v_scale", "heads_k", "q_ld", "k_ld"]),
        "AttnB200MlaShape": (lib.MlaShape, ["dim_v"]),
        "AttnB200SoftmaxBwdArgs": (lib.SoftmaxBwdArgs, ["lse", "dv", "dim_v", "scale", "q_stride", "dv_stride", "workspace_bytes",
                                                        "mask_left", "mask_right", "mask_bits_q", "mask_bits_kv", "mask_tiles_q", "mask_tiles_kv"]),
        "AttnB200ElementwiseBwdArgs": (lib.ElementwiseBwdArgs, ["d_o", "dv", "mask_kind", "q_stride", "custom", "mask_left",
                                                                "mask_bits_q", "mask_bits_kv", "mask_tiles_kv"]),
        "AttnB200MlaArgs": (lib.MlaArgs, ["kv_rope", "o", "workspace_bytes", "shape", "scale", "seq_lens", "block_table",
                                          "block_table_stride", "page_size", "num_pages"]),
    }
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "attn_b200.h"', "int main(void) {"]
    for name, (_, fields) in probes.items():
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for f in fields:
            lines.append(f'  printf("{name}.{f} %zu\\n", offsetof({name}, {f}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "probe.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "probe"
    subprocess.run(["gcc", "-I", os.path.dirname(HEADER), "-o", str(exe), str(src)], check=True)
    seen = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for name, (mirror, fields) in probes.items():
        assert int(seen[name]) == ctypes.sizeof(mirror), name
        for f in fields:
            assert int(seen[f"{name}.{f}"]) == getattr(mirror, f).offset, f"{name}.{f}"


def test_version(native_lib):
    assert native_lib.attn_b200_version() >= 100


def test_null_args_rejected_without_gpu(native_lib):
    assert native_lib.attn_b200_parallel_fwd(None, None) == -1
