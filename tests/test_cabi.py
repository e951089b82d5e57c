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


def test_struct_sizes_match_header(native_lib):
    # layout cross-check of the ctypes mirrors against sizeof() computed from the field list
    assert ctypes.sizeof(lib.ParallelArgs) == 8 * 4 + 8 * 4 + 4 * 6 + 8 * 12 + 4 * 4 + 4 * 8 + 8 * 4 + 8 * 16
    assert ctypes.sizeof(lib.MlaShape) == 20


def test_version(native_lib):
    assert native_lib.attn_b200_version() >= 100


def test_null_args_rejected_without_gpu(native_lib):
    assert native_lib.attn_b200_parallel_fwd(None, None) == -1
