"""Build-and-cache of functor libraries: one small shared library per
(functor source, dim_qk, dim_v, dtype), compiled with nvcc for sm_100a and
loaded with ctypes.

Takes the place of the reference's generated-code caches
(attention_engine/attn_engine/attn_engine.py:380-393: md5-keyed python files;
core/template/cute_template/flash_attn_interface.py:93-123: torch cpp_extension
JIT).  The cache lives inside the package directory so that libraries built on
a machine without a GPU travel with the source tree; the key covers the
generated source, the kernel headers and the compiler version.  A library is
written under a temporary name and renamed, so concurrent builders are safe.
"""

from __future__ import annotations

import ctypes as C
import functools
import hashlib
import os
import subprocess

from core.native import lib as native

JIT_DIR = os.environ.get("ATTN_B200_CACHE_DIR") or os.path.join(os.path.dirname(native.CSRC_DIR), "_jit")
VERBOSE = bool(int(os.environ.get("ATTN_B200_VERBOSE", "0")))

_loaded: dict[str, C.CDLL] = {}


@functools.lru_cache(maxsize=1)
def _toolchain_fingerprint() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(native.CSRC_DIR)):
        if name.endswith(".cuh"):
            with open(os.path.join(native.CSRC_DIR, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    with open(os.path.join(native.INCLUDE_DIR, "attn_b200.h"), "rb") as f:
        h.update(f.read())
    try:
        out = subprocess.run(["nvcc", "--version"], capture_output=True, text=True).stdout
    except FileNotFoundError:
        out = "no-nvcc"
    h.update(out.encode())
    return h.hexdigest()[:16]


def library_path(source: str) -> str:
    key = hashlib.sha256((source + _toolchain_fingerprint()).encode()).hexdigest()[:24]
    return os.path.join(JIT_DIR, f"functor_{key}.so")


def build(source: str, force: bool = False) -> str:
    """Compile ``source`` (a translation unit from core.lower.functor) unless cached."""
    path = library_path(source)
    if os.path.exists(path) and not (force or os.environ.get("ATTN_B200_FORCE_REBUILD")):
        return path
    os.makedirs(JIT_DIR, exist_ok=True)
    cu = path[:-3] + ".cu"
    with open(cu, "w") as f:
        f.write(source)
    tmp = path + f".tmp{os.getpid()}"
    cmd = ["nvcc", *native.NVCC_ARCH_FLAGS, *native.NVCC_COMMON, "-I", native.CSRC_DIR, "-o", tmp, cu]
    if VERBOSE:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if VERBOSE and r.stdout:
        print(r.stdout)
    if r.returncode != 0:
        raise native.NativeError(f"nvcc failed for generated functor {cu}:\n{r.stdout}")
    os.replace(tmp, path)
    return path


def load(source: str):
    """Return the bound ``attn_b200_parallel_fwd_jit`` of the library for ``source``."""
    path = build(source)
    if path not in _loaded:
        dll = C.CDLL(path)
        fn = dll.attn_b200_parallel_fwd_jit
        fn.restype = C.c_int
        fn.argtypes = [C.POINTER(native.ParallelArgs), C.c_void_p, C.c_void_p]
        _loaded[path] = dll
    return _loaded[path].attn_b200_parallel_fwd_jit


def load_backward(source: str):
    """Return the bound ``attn_b200_elementwise_bwd_jit`` of the library for ``source`` (a translation unit from
    core.lower.derivative), compiling it first if it is not cached."""
    path = build(source)
    if path not in _loaded:
        _loaded[path] = C.CDLL(path)
    fn = _loaded[path].attn_b200_elementwise_bwd_jit
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(native.ElementwiseBwdArgs), C.c_void_p, C.c_void_p]
    return fn
