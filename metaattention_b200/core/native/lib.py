"""ctypes binding of libattn_b200.so (the C ABI declared in include/attn_b200.h).

This is the only place where Python touches the native library.  There is no
fallback: if the library is missing or an entry point fails, the call raises.
Tensors are passed as raw device pointers + element strides; kernels run on
the current CUDA stream of the current device, as the reference's native
entry points do (core/template/cute_template_kvshared/flash_api.cpp:46-47,133,188).
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC_DIR = os.path.join(_PKG_DIR, "csrc")
INCLUDE_DIR = os.path.join(os.path.dirname(_PKG_DIR), "include")
LIB_PATH = os.path.join(_PKG_DIR, "libattn_b200.so")

NVCC_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]

MAX_CUSTOM = 4
MAX_ROWSCALES = 4

OK = 0
ERRORS = {
    -1: "invalid argument",
    -2: "unsupported shape / dtype / stride",
    -3: "CUDA launch error",
    -4: "device-side wait timed out",
    -5: "workspace missing or too small",
    -6: "problem needs more scratch than the library's built-in static array holds",
}

DTYPE_CODES = {torch.float16: 0, torch.bfloat16: 1}
DTYPE_OUT_SAME, DTYPE_OUT_FP32 = 0, 2
MASK_NONE, MASK_CAUSAL, MASK_BAND = 0, 1, 2
MASK_BITS = 3            # backward only: any mask without batch / head dependence, as keep bits
MASK_OPEN = 0x3fffffff   # mask_left / mask_right of a band side without a bound
FUNCTOR_SOFTMAX = 0


class NativeError(RuntimeError):
    pass


class ParallelArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
        ("final_rowscales", C.c_void_p * MAX_ROWSCALES),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32),
        ("dim_qk", C.c_int32), ("dim_v", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3),
        ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("dtype", C.c_int32), ("mask_kind", C.c_int32), ("functor", C.c_int32), ("heads_kv", C.c_int32),
        ("fparams", C.c_float * 8),
        ("custom", C.c_void_p * MAX_CUSTOM),
        ("custom_stride", (C.c_int64 * 4) * MAX_CUSTOM),
        ("mask_left", C.c_int32), ("mask_right", C.c_int32),
        ("num_splits", C.c_int32), ("reserved", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("tile_keep", C.c_void_p), ("tile_partial", C.c_void_p), ("tile_mask_base", C.c_void_p), ("elem_mask", C.c_void_p),
        ("sparse_batch", C.c_int32), ("sparse_heads", C.c_int32), ("elem_mask_rows", C.c_int32), ("reserved2", C.c_int32),
    ]


class LinearArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("log_decay", C.c_void_p), ("o", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("seq", C.c_int32), ("dim_qk", C.c_int32), ("dim_v", C.c_int32),
        ("dtype", C.c_int32), ("normalize", C.c_int32), ("q_scale", C.c_float), ("norm_eps", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("dtype_out", C.c_int32), ("precise", C.c_int32),
        ("v_scale", C.c_void_p), ("heads_q", C.c_int32), ("heads_k", C.c_int32), ("q_ld", C.c_int32), ("k_ld", C.c_int32),
    ]


class SoftmaxBwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
        ("lse", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("heads_kv", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32),
        ("dim_qk", C.c_int32), ("dim_v", C.c_int32), ("dtype", C.c_int32), ("mask_kind", C.c_int32), ("scale", C.c_float),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("do_stride", C.c_int64 * 3), ("dq_stride", C.c_int64 * 3), ("dk_stride", C.c_int64 * 3), ("dv_stride", C.c_int64 * 3),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64), ("mask_left", C.c_int32), ("mask_right", C.c_int32),
        ("mask_bits_q", C.c_void_p), ("mask_bits_kv", C.c_void_p), ("mask_tiles_q", C.c_void_p), ("mask_tiles_kv", C.c_void_p),
    ]


class ElementwiseBwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("d_o", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("batch", C.c_int32), ("heads", C.c_int32), ("heads_kv", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32),
        ("dim_qk", C.c_int32), ("dim_v", C.c_int32), ("dtype", C.c_int32), ("mask_kind", C.c_int32), ("reserved", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3), ("do_stride", C.c_int64 * 3),
        ("dq_stride", C.c_int64 * 3), ("dk_stride", C.c_int64 * 3), ("dv_stride", C.c_int64 * 3),
        ("custom", C.c_void_p * MAX_CUSTOM), ("mask_left", C.c_int32), ("mask_right", C.c_int32),
        ("mask_bits_q", C.c_void_p), ("mask_bits_kv", C.c_void_p), ("mask_tiles_q", C.c_void_p), ("mask_tiles_kv", C.c_void_p),
    ]


class MlaShape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("heads_q", C.c_int32), ("seq_kv", C.c_int32),
                ("dim_qk", C.c_int32), ("dim_v", C.c_int32)]


class MlaArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("kv", C.c_void_p), ("q_rope", C.c_void_p), ("kv_rope", C.c_void_p),
        ("q_stride", C.c_int64 * 2), ("kv_stride", C.c_int64 * 2),
        ("q_rope_stride", C.c_int64 * 2), ("kv_rope_stride", C.c_int64 * 2),
        ("o", C.c_void_p), ("lse", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("shape", MlaShape), ("num_splits", C.c_int32), ("dtype", C.c_int32), ("scale", C.c_float),
        ("seq_lens", C.c_void_p), ("block_table", C.c_void_p), ("block_table_stride", C.c_int64),
        ("page_size", C.c_int32), ("num_pages", C.c_int32),
        ("sched_meta", C.c_void_p), ("sched_num_splits", C.c_void_p), ("sched_parts", C.c_int32), ("reserved", C.c_int32),
    ]


# symbol name -> (restype, argtypes); must list every function of include/attn_b200.h
SIGNATURES = {
    "attn_b200_parallel_fwd": (C.c_int, [C.POINTER(ParallelArgs), C.c_void_p]),
    "attn_b200_parallel_workspace_bytes": (C.c_int64, [C.POINTER(ParallelArgs)]),
    "attn_b200_decode_tiles_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32]),
    "attn_b200_decode_tiles": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_void_p, C.c_int64, C.c_void_p]),
    "attn_b200_linear_fwd": (C.c_int, [C.POINTER(LinearArgs), C.c_void_p]),
    "attn_b200_rows_copy16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                        C.c_void_p]),
    "attn_b200_rows_sum_cast": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int32,
                                          C.c_int32, C.c_void_p]),
    "attn_b200_linear_workspace_bytes": (C.c_int64, [C.POINTER(LinearArgs)]),
    "attn_b200_softmax_bwd": (C.c_int, [C.POINTER(SoftmaxBwdArgs), C.c_void_p]),
    "attn_b200_softmax_bwd_workspace_bytes": (C.c_int64, [C.POINTER(SoftmaxBwdArgs)]),
    "attn_b200_mla_plan": (C.c_int, [C.POINTER(MlaShape), C.c_int32, C.POINTER(C.c_int32)]),
    "attn_b200_mla_workspace_bytes": (C.c_int64, [C.POINTER(MlaShape), C.c_int32]),
    "attn_b200_mla_num_parts": (C.c_int32, [C.c_int32, C.c_int32]),
    "attn_b200_mla_metadata": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "attn_b200_mla_decode": (C.c_int, [C.POINTER(MlaArgs), C.c_void_p]),
    "attn_b200_mla_decode_static": (C.c_int, [C.POINTER(MlaArgs), C.c_void_p, C.c_void_p]),
    "attn_b200_last_device_status": (C.c_int, [C.c_int32, C.POINTER(C.c_int32)]),
    "attn_b200_device_status_word": (C.c_int, [C.c_int32, C.POINTER(C.c_void_p)]),
    "attn_b200_version": (C.c_int, []),
}

_lib = None


def library_sources() -> list[str]:
    return [os.path.join(CSRC_DIR, f) for f in ("attn_b200.cu", "mla_decode.cu", "linear_fwd.cu", "softmax_bwd.cu", "row_ops.cu")]


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile libattn_b200.so for sm_100a with nvcc (cross-compiles without a GPU)."""
    srcs = library_sources()
    deps = srcs + [os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cuh")] + \
        [os.path.join(INCLUDE_DIR, "attn_b200.h")]
    if not force and os.path.exists(LIB_PATH) and \
            os.path.getmtime(LIB_PATH) >= max(os.path.getmtime(d) for d in deps):
        return LIB_PATH
    objs = []
    procs = []
    for src in srcs:
        obj = src[:-3] + ".o"
        cmd = ["nvcc", *NVCC_ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
               "-I", INCLUDE_DIR, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for cmd, pr in procs:
        out, _ = pr.communicate()
        if verbose and out:
            print(out)
        if pr.returncode != 0:
            raise NativeError(f"nvcc failed: {' '.join(cmd)}\n{out}")
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    link = ["nvcc", *NVCC_ARCH_FLAGS, "-shared", "-o", tmp, *objs]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise NativeError(f"link failed: {' '.join(link)}\n{r.stdout}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def bind(lib: C.CDLL, names=None) -> C.CDLL:
    for name in (names or SIGNATURES):
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = SIGNATURES[name]
    return lib


def load_library() -> C.CDLL:
    """Load (once) the native library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        path = os.environ.get("ATTN_B200_LIBRARY", LIB_PATH)  # an alternative build of the same ABI
        if not os.path.exists(path):
            raise NativeError(
                f"{path} not found: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "from the repository root (there is no non-native fallback)")
        _lib = bind(C.CDLL(path))
    return _lib


def check(rc: int, what: str):
    if rc != OK:
        raise NativeError(f"{what} failed: {ERRORS.get(rc, 'error')} (code {rc})")


def current_stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def device_status_word(device: int) -> int:
    out = C.c_void_p()
    check(load_library().attn_b200_device_status_word(device, C.byref(out)), "attn_b200_device_status_word")
    return out.value


def last_device_status(device: int | None = None) -> int:
    """Synchronise and return (then clear) the device status word: 0, or
    100 + id of the device-side wait that gave up."""
    if device is None:
        device = torch.cuda.current_device()
    out = C.c_int32(0)
    check(load_library().attn_b200_last_device_status(device, C.byref(out)), "attn_b200_last_device_status")
    return out.value


def _strides_bsh(t: torch.Tensor):
    """Element strides (batch, seq, head) of a [B, S, H, D] tensor view."""
    return (t.stride(0), t.stride(1), t.stride(2))


def fill_parallel_args(q, k, v, o, *, mask_kind: int, functor: int = 0, fparams=(), final_rowscales=(),
                       custom=(), custom_strides=(), mask_band=(MASK_OPEN, MASK_OPEN), num_splits: int = 1,
                       workspace=None, sparse=None) -> ParallelArgs:
    """q,k: [B,S,H,D]; v,o: [B,S,H,Dv] CUDA tensors (any strides with a contiguous last dim)."""
    for t in (q, k, v, o):
        if not t.is_cuda:
            raise NativeError("parallel forward needs CUDA tensors")
        if t.stride(-1) != 1:
            raise NativeError("last dimension must be contiguous")
    if q.dtype not in DTYPE_CODES or k.dtype != q.dtype or v.dtype != q.dtype or o.dtype != q.dtype:
        raise NativeError(f"q, k, v, o must share dtype float16 or bfloat16 (got {q.dtype}, {k.dtype}, {v.dtype}, {o.dtype})")
    a = ParallelArgs()
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    for i, t in enumerate(final_rowscales):
        a.final_rowscales[i] = t.data_ptr() if t is not None else None
    B, Sq, H, D = q.shape
    a.batch, a.heads, a.seq_q, a.seq_kv, a.dim_qk, a.dim_v = B, H, Sq, k.shape[1], D, v.shape[3]
    if k.shape[2] != v.shape[2] or H % k.shape[2] != 0:
        raise NativeError(f"k and v need the same number of heads, a divisor of the query heads (got {H}, {k.shape[2]}, {v.shape[2]})")
    a.heads_kv = k.shape[2]
    a.q_stride[:] = _strides_bsh(q)
    a.k_stride[:] = _strides_bsh(k)
    a.v_stride[:] = _strides_bsh(v)
    a.o_stride[:] = _strides_bsh(o)
    a.dtype = DTYPE_CODES[q.dtype]
    a.mask_kind = mask_kind
    a.mask_left, a.mask_right = int(mask_band[0]), int(mask_band[1])
    a.num_splits = int(num_splits)
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    if sparse is not None:   # dict from core.lower.sparse: device tensors + extents
        a.tile_keep, a.tile_partial = sparse["keep"].data_ptr(), sparse["partial"].data_ptr()
        a.tile_mask_base = sparse["mask_base"].data_ptr() if sparse.get("mask_base") is not None else None
        a.elem_mask = sparse["elem_mask"].data_ptr() if sparse.get("elem_mask") is not None else None
        a.sparse_batch, a.sparse_heads, a.elem_mask_rows = sparse["batch"], sparse["heads"], sparse["mask_rows"]
    a.functor = functor
    for i, f in enumerate(fparams):
        a.fparams[i] = float(f)
    for i, t in enumerate(custom):
        a.custom[i] = t.data_ptr()
        for j, s in enumerate(custom_strides[i]):
            a.custom_stride[i][j] = int(s)
    return a


def decode_tiles(block_mask, cache_seqlens, batch: int, heads_kv: int, seq_kv: int, block_size: int, device) -> dict:
    """Sparse-walk description (see fill_parallel_args ``sparse``) of a block-sparse, variable-length decode, built
    on the device by attn_b200_decode_tiles.  block_mask: bool/uint8 [batch, heads_kv, blocks] or None;
    cache_seqlens: int32 [batch] or None."""
    lib = load_library()
    tiles = (seq_kv + 127) // 128
    words = (tiles + 31) // 32
    bh = batch * heads_kv
    out = torch.empty(int(lib.attn_b200_decode_tiles_bytes(batch, heads_kv, seq_kv)) // 4, dtype=torch.int32, device=device)
    n_blocks = 0
    if block_mask is not None:
        if block_mask.dim() != 3 or block_mask.shape[0] != batch or block_mask.shape[1] != heads_kv:
            raise NativeError(f"block_mask must be [batch, kv heads, blocks] = [{batch}, {heads_kv}, *], got {tuple(block_mask.shape)}")
        block_mask = block_mask.to(device=device).contiguous()
        block_mask = block_mask.view(torch.uint8) if block_mask.dtype == torch.bool else block_mask.to(torch.uint8)
        n_blocks = block_mask.shape[2]
    if cache_seqlens is not None:
        if cache_seqlens.numel() != batch:
            raise NativeError(f"cache_seqlens must hold one length per sequence ({batch}), got {cache_seqlens.numel()}")
        cache_seqlens = cache_seqlens.to(device=device, dtype=torch.int32).contiguous()
    check(lib.attn_b200_decode_tiles(block_mask.data_ptr() if block_mask is not None else None,
                                     cache_seqlens.data_ptr() if cache_seqlens is not None else None,
                                     batch, heads_kv, n_blocks, int(block_size), seq_kv, out.data_ptr(), out.numel() * 4,
                                     current_stream_ptr()), "attn_b200_decode_tiles")
    col = out[:bh * tiles * 4]
    keep = out[bh * tiles * 4:bh * tiles * 4 + bh * words]
    part = out[bh * tiles * 4 + bh * words:]
    return {"keep": keep, "partial": part, "mask_base": None, "elem_mask": col, "batch": batch, "heads": heads_kv,
            "mask_rows": 0, "_owner": (out, block_mask, cache_seqlens)}


def rows_copy(src, col0: int = 0, width: int | None = None, reverse: bool = False):
    """Contiguous copy of columns [col0, col0 + width) of a 16-bit tensor [..., seq, cols], the rows of every sequence in
    reversed order if asked (attn_b200_rows_copy16): one pass for what torch does as flip + slice + contiguous."""
    if not src.is_cuda:
        raise NativeError("rows_copy needs a CUDA tensor: there is no CPU path")
    if src.dtype not in DTYPE_CODES:
        raise NativeError("rows_copy moves float16 / bfloat16 tensors")
    src = src.contiguous()
    cols, seq = src.shape[-1], src.shape[-2]
    width = cols - col0 if width is None else width
    dst = torch.empty(src.shape[:-1] + (width,), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        check(load_library().attn_b200_rows_copy16(src.data_ptr(), dst.data_ptr(), src.numel() // (seq * cols), seq, cols, col0, width,
                                                   1 if reverse else 0, current_stream_ptr()), "attn_b200_rows_copy16")
    return dst


def rows_sum_cast(a, b, dtype, reverse: bool = False):
    """a (+ b), fp32 [..., seq, cols], rounded to ``dtype`` with the rows of every sequence reversed if asked
    (attn_b200_rows_sum_cast)."""
    if not a.is_cuda:
        raise NativeError("rows_sum_cast needs CUDA tensors: there is no CPU path")
    a = a.contiguous()
    b = None if b is None else b.contiguous()
    cols, seq = a.shape[-1], a.shape[-2]
    dst = torch.empty(a.shape, dtype=dtype, device=a.device)
    with torch.cuda.device(a.device):
        check(load_library().attn_b200_rows_sum_cast(a.data_ptr(), None if b is None else b.data_ptr(), dst.data_ptr(),
                                                     DTYPE_CODES[dtype], a.numel() // (seq * cols), seq, cols, 1 if reverse else 0,
                                                     current_stream_ptr()), "attn_b200_rows_sum_cast")
    return dst


def _over_dim_v_slices(run, q, k, v, d_o, o=None):
    """dim_v a multiple of dim_qk (the 128 / 256 of the reference's suite, testing/test.py:55): the backward is linear in
    dP = dO V^T and in delta = rowsum(dO o O), both sums over the columns of v, and dV's columns are independent, so it
    is one kernel run per dim_qk-wide column slice of (v, o, dO) — each recomputing P — with dQ and dK added up in fp32."""
    D, Dv = q.shape[-1], v.shape[-1]
    if Dv == D:
        return run(q, k, v, d_o, o)
    if Dv % D != 0:
        raise NativeError(f"the backward covers dim_v = a multiple of dim_qk (got {D} / {Dv})")
    dq = dk = None
    dvs = []
    for c in range(0, Dv, D):
        part = run(q, k, v[..., c:c + D], d_o[..., c:c + D], None if o is None else o[..., c:c + D])
        dq = part[0].float() if dq is None else dq + part[0].float()
        dk = part[1].float() if dk is None else dk + part[1].float()
        dvs.append(part[2])
    return dq.to(q.dtype), dk.to(k.dtype), torch.cat(dvs, dim=-1)


def softmax_bwd(q, k, v, o, lse, d_o, scale: float, mask_kind: int, mask_band=(MASK_OPEN, MASK_OPEN), mask_bits=None):
    """(dq, dk, dv) of softmax attention from the forward's o and lse [B, H, Sq] and the gradient of o
    (attn_b200_softmax_bwd: mask NONE, CAUSAL or BAND with ``mask_band`` = (left, right); head dims 128 / 128 and
    64 / 64; dim_v a larger multiple of dim_qk as one run per column slice).  ``mask_bits`` = (bits_q, bits_kv[, tiles_q,
    tiles_kv]), the keep matrix of a general mask and its transpose as device int32 tensors and, optionally, the bitmaps of
    the tile pairs that keep anything (core/lower/sparse.py:mask_bit_matrices), replaces the mask kind by MASK_BITS."""
    for t in (q, k, v, o, d_o, lse):
        if not t.is_cuda:
            raise NativeError("the backward kernel needs CUDA tensors: there is no CPU path")
    if d_o.stride(-1) != 1:
        d_o = d_o.contiguous()
    return _over_dim_v_slices(lambda q_, k_, v_, do_, o_: _softmax_bwd_one(q_, k_, v_, o_, lse, do_, scale, mask_kind, mask_band, mask_bits),
                              q, k, v, d_o, o)


def _set_mask_bits(a, mask_bits, q, k):
    """Fills mask_kind / mask_bits_* of a backward argument struct from (bits_q, bits_kv) after checking their shapes."""
    bq, bk = mask_bits[:2]
    nq, nk = -(-q.shape[1] // 128), -(-k.shape[1] // 128)
    want = [(bq, (nq * 128, nk, 4)), (bk, (nk * 128, nq, 4))]
    if len(mask_bits) == 4:   # + bitmaps of the tiles that keep anything
        want += [(mask_bits[2], (nq, -(-nk // 32))), (mask_bits[3], (nk, -(-nq // 32)))]
    for t, shape in want:
        if not (t.is_cuda and t.dtype == torch.int32 and t.is_contiguous() and tuple(t.shape) == shape):
            raise NativeError(f"mask bits: expected a contiguous CUDA int32 tensor of shape {shape}, got {tuple(t.shape)}")
    a.mask_kind, a.mask_bits_q, a.mask_bits_kv = MASK_BITS, bq.data_ptr(), bk.data_ptr()
    if len(mask_bits) == 4:
        a.mask_tiles_q, a.mask_tiles_kv = mask_bits[2].data_ptr(), mask_bits[3].data_ptr()


def _softmax_bwd_one(q, k, v, o, lse, d_o, scale: float, mask_kind: int, mask_band, mask_bits=None):
    for t in (q, k, v, o):
        if t.stride(-1) != 1:
            raise NativeError("last dimension must be contiguous")
    if q.dtype not in DTYPE_CODES or any(t.dtype != q.dtype for t in (k, v, o, d_o)):
        raise NativeError("q, k, v, o, d_o must share dtype float16 or bfloat16")
    lse = lse.contiguous().float()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if dq.stride(-1) != 1 or dk.stride(-1) != 1 or dv.stride(-1) != 1:
        dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (q, k, v))
    a = SoftmaxBwdArgs()
    a.q, a.k, a.v, a.o, a.d_o, a.lse = (t.data_ptr() for t in (q, k, v, o, d_o, lse))
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    B, Sq, H, D = q.shape
    a.batch, a.heads, a.heads_kv, a.seq_q, a.seq_kv, a.dim_qk, a.dim_v = B, H, k.shape[2], Sq, k.shape[1], D, v.shape[3]
    a.dtype, a.mask_kind, a.scale = DTYPE_CODES[q.dtype], mask_kind, float(scale)
    a.mask_left, a.mask_right = int(mask_band[0]), int(mask_band[1])
    if mask_bits is not None:
        _set_mask_bits(a, mask_bits, q, k)
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", d_o), ("dq", dq), ("dk", dk), ("dv", dv)):
        getattr(a, name + "_stride")[:] = _strides_bsh(t)
    lib = load_library()
    need = lib.attn_b200_softmax_bwd_workspace_bytes(C.byref(a))
    if need < 0:
        raise NativeError("attn_b200_softmax_bwd_workspace_bytes: bad arguments")
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    with torch.cuda.device(q.device):
        check(lib.attn_b200_softmax_bwd(C.byref(a), current_stream_ptr()), "attn_b200_softmax_bwd")
    return dq, dk, dv


def elementwise_bwd(fn, q, k, v, d_o, mask_kind: int, custom=(), mask_band=(MASK_OPEN, MASK_OPEN), mask_bits=None):
    """(dq, dk, dv) of an elementwise program through its functor library's ``attn_b200_elementwise_bwd_jit`` (``fn``);
    ``custom``: the program's fp32 scalar inputs, as device tensors.  dim_v may be a multiple of dim_qk."""
    for t in (q, k, v, d_o, *custom):
        if not t.is_cuda:
            raise NativeError("the backward kernel needs CUDA tensors: there is no CPU path")
    if d_o.stride(-1) != 1:
        d_o = d_o.contiguous()
    return _over_dim_v_slices(lambda q_, k_, v_, do_, o_: _elementwise_bwd_one(fn, q_, k_, v_, do_, mask_kind, custom, mask_band, mask_bits),
                              q, k, v, d_o)


def _elementwise_bwd_one(fn, q, k, v, d_o, mask_kind: int, custom, mask_band, mask_bits=None):
    if q.dtype not in DTYPE_CODES or any(t.dtype != q.dtype for t in (k, v, d_o)):
        raise NativeError("q, k, v, d_o must share dtype float16 or bfloat16")
    dq, dk, dv = (torch.empty(t.shape, dtype=t.dtype, device=t.device) for t in (q, k, v))
    custom = [t.to(device=q.device, dtype=torch.float32).contiguous() for t in custom]
    a = ElementwiseBwdArgs()
    a.q, a.k, a.v, a.d_o = (t.data_ptr() for t in (q, k, v, d_o))
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    B, Sq, H, D = q.shape
    a.batch, a.heads, a.heads_kv, a.seq_q, a.seq_kv, a.dim_qk, a.dim_v = B, H, k.shape[2], Sq, k.shape[1], D, v.shape[3]
    a.dtype, a.mask_kind = DTYPE_CODES[q.dtype], mask_kind
    a.mask_left, a.mask_right = int(mask_band[0]), int(mask_band[1])
    if mask_bits is not None:
        _set_mask_bits(a, mask_bits, q, k)
    for name, t in (("q", q), ("k", k), ("v", v), ("do", d_o), ("dq", dq), ("dk", dk), ("dv", dv)):
        getattr(a, name + "_stride")[:] = _strides_bsh(t)
    for i, t in enumerate(custom):
        a.custom[i] = t.data_ptr()
    with torch.cuda.device(q.device):
        status = device_status_word(q.device.index)
        check(fn(C.byref(a), current_stream_ptr(), status), "attn_b200_elementwise_bwd_jit")
    return dq, dk, dv


def parallel_fwd(args: ParallelArgs):
    check(load_library().attn_b200_parallel_fwd(C.byref(args), current_stream_ptr()), "attn_b200_parallel_fwd")
