"""``AttentionEngine`` / ``OnlineFunc``: the user-facing API of the reference
(attention_engine/attn_engine/attn_engine.py:16-105 ``OnlineFunc``, :108-116
constructor, :227-343 pattern selection, :399-408 ``__call__``) on top of the
native sm_100a backend.

What happens at construction: the shapes in ``qkv_meta`` select a pattern
(same rules as the reference), the user's ``score_mod`` / ``online_func`` are
traced once into a DAG, ``mask_mod`` is classified, and the DAG is either
recognised as a built-in functor of ``libattn_b200.so`` or lowered to a C++
device functor that is compiled (and cached) for the forward-kernel template.
Tuning arguments are accepted and ignored: kernel configurations are fixed.

There is no CPU or eager fallback: calling an engine needs CUDA tensors, the
native library and an sm_100a device.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from core.lower import functor as functor_lowering
from core.lower import sparse as sparse_lowering
from core.lower import derivative
from core.lower.trace import probe_softmax_scale, trace_parallel
from core.native import jit as native_jit
from core.native import lib as native
from core.transform.core import CustomIO, SymbolicArray, SymbolScalar, Var, _eval_mask_2d, \
    mask_depends_on_batch_head
from core.lower.trace import custom_axes


class OnlineFunc:
    """Base class of user-defined online functions (same protocol as the reference).

    ``__init__`` declares ``online_rowscales`` (running per-row values, each a
    ``SymbolScalar(name, Var(initial_value_string))``) and ``final_rowscales``
    (per-row outputs).  ``online_fwd`` maps one score tile and the running row
    scales to (new scores, new row scales, o_scale); ``online_fwd_epilogue``
    maps the accumulator and the row scales to (output, final row scales);
    ``combine`` gives the per-split output scale of a split-KV kernel.
    ``forward`` / ``backward`` describe the backward recomputation and are not
    used by the forward-only backend.
    """

    def __init__(self, online_rowscales: dict, final_rowscales: dict, external_fwd_tensors: CustomIO):
        self.online_rowscales = online_rowscales
        self.final_rowscales = final_rowscales
        self.vars = {"scores": SymbolicArray(), "o_scale": None}
        self.external_fwd_tensors = external_fwd_tensors
        self.doosum_rowscales = SymbolicArray("doosum", Var("doosum"), shape_idx=["block_M"])

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        return scores, online_rowscales, SymbolScalar("o_scale", Var("1"))

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, online_rowscales

    @staticmethod
    def forward(scores, final_rowscales, b, h, q_idx, kv_idx):
        return scores

    @staticmethod
    def backward(dp, scores, final_rowscales, doosum_rowscales, b, h, q_idx, kv_idx):
        return dp

    @staticmethod
    def combine(final_rowscales):
        return SymbolScalar("o_scale", Var("1"))


class _ForwardOnly(torch.autograd.Function):
    """Keeps autograd graphs well-formed: the forward runs the native kernel,
    the backward states clearly that it does not exist for this program."""

    @staticmethod
    def forward(ctx, runner, *tensors):
        return runner(*[t.detach() for t in tensors])

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("the B200-native backend has a backward pass for softmax attention (score_mod = scale, "
                                  "the softmax online_func) and for elementwise programs (no row scales, scalar custom "
                                  "inputs), with no mask or a causal mask and head dims 128 / 128 or 64 / 64")


class _SoftmaxAttention(torch.autograd.Function):
    """Softmax attention with its native backward (attn_b200_softmax_bwd), the counterpart of the reference's
    ``_attention`` autograd function (core/template/tl_template/attn/attn_tl.py:654-694): the forward keeps o and the
    log-sum-exp, the backward recomputes the probabilities from them."""

    @staticmethod
    def forward(ctx, engine, q, k, v):
        q, k, v = q.detach(), k.detach(), v.detach()
        o = engine._run_parallel_impl(q, k, v)
        lse = engine.last_final_rowscales[engine.final_names[0]]
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.engine = engine
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        eng = ctx.engine
        dq, dk, dv = native.softmax_bwd(q, k, v, o, lse, d_o.to(q.dtype), eng._fparams[0], eng.mask_kind, eng.mask_band,
                                        eng._mask_bits(q.device))
        return None, dq, dk, dv


class _ElementwiseAttention(torch.autograd.Function):
    """An elementwise program (P = f(q.k): sigmoid, relu attention ...) with the backward derived from its traced
    score_mod (core/lower/derivative.py) and compiled on first use."""

    @staticmethod
    def forward(ctx, engine, n_custom, q, k, v, *custom):
        q, k, v = q.detach(), k.detach(), v.detach()
        custom = tuple(t.detach() if isinstance(t, torch.Tensor) else t for t in custom)
        o = engine._run_parallel_impl(q, k, v, *custom)
        ctx.save_for_backward(q, k, v, *custom)
        ctx.engine = engine
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, *custom = ctx.saved_tensors
        eng = ctx.engine
        if eng._bwd_fn is None:
            eng._bwd_fn = native_jit.load_backward(eng._bwd_source)
        dq, dk, dv = native.elementwise_bwd(eng._bwd_fn, q, k, v, d_o.to(q.dtype), eng.mask_kind, custom, eng.mask_band,
                                            eng._mask_bits(q.device))
        return (None, None, dq, dk, dv) + (None,) * len(custom)


def plan_kv_splits(batch: int, heads: int, q_len: int, kv_len: int, device) -> int:
    """KV splits for the forward kernel: 1 unless the (query tile pair, head, batch) grid fills less than half of
    the SMs; then as many as fit, each keeping at least four 128-row KV tiles (a split re-reads Q and adds a
    combine pass)."""
    ctas = batch * heads * ((q_len + 255) // 256)
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    kv_tiles = (kv_len + 127) // 128
    if 2 * ctas > sms or kv_tiles < 8:
        return 1
    return max(1, min(sms // ctas, kv_tiles // 4, 65535 // max(batch, 1)))


MASK_GENERAL = -1   # classify_mask: not a band, or different per batch / head: runs as a block-sparse walk


def classify_mask(mask_mod, B: int, H: int, q_len: int, kv_len: int):
    """(mask kind, (left, right)) for a ``mask_mod(b, h, q_idx, kv_idx)``: MASK_NONE, MASK_CAUSAL,
    MASK_BAND = keep q_idx - left <= kv_idx <= q_idx + right (sliding windows; MASK_OPEN = no bound on
    that side), or MASK_GENERAL for everything else (any other pattern, and masks that use the batch or head
    index), which the engine turns into a block-sparse walk (core/lower/sparse.py).  The mask is evaluated on CPU for one (b, h) over the [q_len, kv_len] grid (never the
    B*H*S*S tensor the reference materialises at core/lower/lower.py:729) and compared with the band it
    suggests; the kernel then skips the KV tiles outside the band, which is what the reference's block
    mask does for it (core/transform/core.py:492-506)."""
    open_band = (native.MASK_OPEN, native.MASK_OPEN)
    if mask_mod is None:
        return native.MASK_NONE, open_band
    if mask_depends_on_batch_head(mask_mod, B, H, q_len, kv_len, "cpu"):
        return MASK_GENERAL, open_band
    dense = _eval_mask_2d(mask_mod, 0, 0, q_len, kv_len, "cpu")
    if bool(dense.all()):
        return native.MASK_NONE, open_band
    q = torch.arange(q_len).view(-1, 1)
    kv = torch.arange(kv_len).view(1, -1)
    if torch.equal(dense, kv <= q):
        return native.MASK_CAUSAL, open_band
    if bool(dense.any(dim=1).all()):
        # widest reach of any row to either side of its diagonal; a side that always runs to the edge is open
        first = dense.float().argmax(dim=1)
        last = kv_len - 1 - dense.flip(1).float().argmax(dim=1)
        rows = torch.arange(q_len)
        left = int((rows - first).max())
        right = int((last - rows).max())
        if left >= 0 and right >= 0:
            if bool((first == 0).all()):
                left = native.MASK_OPEN
            if bool((last == kv_len - 1).all()):
                right = native.MASK_OPEN
            if torch.equal(dense, (kv >= q - left) & (kv <= q + right)):
                return native.MASK_BAND, (left, right)
    return MASK_GENERAL, open_band


class AttentionEngine:
    def __init__(self, qkv_meta, custom_fwd_inputs, score_mod, mask_mod, online_func, mask_value="-inf",
                 device=None, backend="tl", tune=False, tune_file="", tune_bwd=False, tune_file_bwd="",
                 infer_mask=True, infer_mask_block_M=128, infer_mask_block_N=128, extern_block_mask=False,
                 use_varlen=False, kv_shared=False):
        if backend not in ("tl", "cute", "cute_v2"):
            raise ValueError(f"unknown backend {backend!r}")
        self.backend = backend          # accepted for source compatibility; every value runs the native kernels
        self.use_varlen = use_varlen
        self.block_mask = None
        self._decode_block = None  # block size of a call-time block_mask (block-sparse, variable-length decode)
        self._sparse_host = None   # block-sparse walk of a general mask_mod (built once, on the CPU)
        self._bwd_source = None    # translation unit of the backward functor library (elementwise programs)
        self._bwd_fn = None
        self._sparse_dev = {}      # its copies by device
        self.kv_splits = None      # None = planned per call (plan_kv_splits); an int forces the split count
        self.qkv_meta = qkv_meta
        self.custom_fwd_inputs = custom_fwd_inputs if custom_fwd_inputs is not None else CustomIO()
        self.last_final_rowscales: dict[str, torch.Tensor] = {}
        q_meta, k_meta, v_meta = qkv_meta
        B, H, Sq, D = q_meta.shape
        Hkv, Skv = v_meta.shape[1], v_meta.shape[2]
        Dv = v_meta.shape[3]
        dtype = q_meta.dtype
        if dtype not in native.DTYPE_CODES:
            raise TypeError(f"dtype {dtype} is not supported: use torch.float16 or torch.bfloat16")
        self.dtype = dtype
        self.pattern = self._select_pattern(Sq, Skv, H, Hkv, kv_shared)
        if self.pattern == "mla_decode":
            from attn_engine.mla import build_mla_decode
            self.attention = build_mla_decode(self, B, H, Hkv, Skv, D, Dv, dtype, backend)
        elif self.pattern == "parallel":
            self._build_parallel(B, H, Sq, D, Dv, dtype, score_mod, mask_mod, online_func, mask_value)
        elif self.pattern in ("gqa", "gqa_decode"):
            # grouped KV heads (the reference's lower_gqa.py / attn_gqa_tl.py and the dense case of its GQA decode):
            # the same forward kernel, query head h reading KV head h / (H / Hkv); K/V of a group are fetched
            # once per query head and mostly hit L2.  With extern_block_mask / use_varlen (examples/sparse_gqa_decode.py)
            # the kept blocks and cache lengths of each call select the KV tiles that are visited.
            if H % Hkv != 0:
                raise NotImplementedError(f"query heads ({H}) must be a multiple of KV heads ({Hkv})")
            if use_varlen or extern_block_mask:
                self._decode_block = int(infer_mask_block_N)
            self._build_parallel(B, H, Sq, D, Dv, dtype, score_mod, mask_mod, online_func, mask_value, kv_len=Skv)
        elif self.pattern == "mha_decode":
            # A few query rows against a long KV (examples/mha_decode.py; the reference lowers it to a split-KV
            # kernel plus OnlineFunc.combine, lower_decode.py:375-449).  The forward kernel takes any
            # q_len != kv_len, streams K/V once per (batch, head) and needs no combine step; with few
            # (batch, head) pairs it leaves SMs idle.
            if use_varlen or extern_block_mask:
                self._decode_block = int(infer_mask_block_N)
            self._build_parallel(B, H, Sq, D, Dv, dtype, score_mod, mask_mod, online_func, mask_value, kv_len=Skv)
        else:
            raise NotImplementedError(
                f"pattern {self.pattern!r} (q_len={Sq}, kv_len={Skv}, heads={H}, kv_heads={Hkv}) is not covered by the "
                "native backend yet: it implements the parallel MHA / GQA forward, dense MHA / GQA decode, chunked linear "
                "attention and MLA decode")

    # ------------------------------------------------------------------
    # pattern selection by shape, as attn_engine.py:227-343 of the reference
    @staticmethod
    def _select_pattern(q_len, kv_len, heads, heads_kv, kv_shared) -> str:
        if kv_shared:
            return "mla_decode"
        if q_len != kv_len and heads > heads_kv:
            return "gqa_decode"
        if q_len != kv_len and heads == heads_kv:
            return "mha_decode"
        if q_len == kv_len and heads == heads_kv:
            return "parallel"
        return "gqa"

    # ------------------------------------------------------------------
    def _build_parallel(self, B, H, S, D, Dv, dtype, score_mod, mask_mod, online_func, mask_value, kv_len=None):
        if (D, Dv) not in ((64, 64), (128, 128), (192, 128)) and not (D in (128, 256) and Dv % 128 == 0):
            raise NotImplementedError(f"head dims (qk={D}, v={Dv}) are not covered by the forward kernel yet "
                                      "(supported: 64/64, 192/128, and 128 or 256 / a multiple of 128)")
        Skv = S if kv_len is None else kv_len
        self.mask_kind, self.mask_band = classify_mask(mask_mod, B, H, S, Skv)
        if self.mask_kind != native.MASK_NONE and self._decode_block is not None:
            raise NotImplementedError("a mask_mod together with a call-time block_mask / cache_seqlens is not supported")
        if self.mask_kind == MASK_GENERAL or (Skv != S and self.mask_kind != native.MASK_NONE):
            # the reference's choice for anything that is not causal (core/lower/lower.py:723-738): block sparsity.
            # KV tiles without a kept position are skipped, partially kept ones carry their element mask.
            self._sparse_host = sparse_lowering.build_block_sparse(mask_mod, B, H, S, Skv)
            self.mask_kind = native.MASK_NONE
        self.sparse_walk = self._sparse_host is not None or self._decode_block is not None
        neg_inf_mask = str(mask_value).strip() in ("-inf", "-float('inf')")
        self._neg_inf_mask = neg_inf_mask
        self.traced = trace_parallel(score_mod, online_func, self.custom_fwd_inputs)
        tr = self.traced
        if len(tr.custom) > native.MAX_CUSTOM:
            raise NotImplementedError(f"at most {native.MAX_CUSTOM} custom inputs are supported")
        if len(tr.final) > native.MAX_ROWSCALES or len(tr.rowscale_in) > native.MAX_ROWSCALES:
            raise NotImplementedError(f"at most {native.MAX_ROWSCALES} row scales are supported")
        self.final_names = list(tr.final.keys())
        self.custom_names = list(tr.custom.keys())
        self._custom_syms = [tr.custom[n] for n in self.custom_names]
        input_ctype = "__nv_bfloat16" if dtype == torch.bfloat16 else "__half"
        self._custom_dtypes = [torch.float32 if functor_lowering.custom_kind(s) == "scalar" else dtype
                               for s in self._custom_syms]

        scale = probe_softmax_scale(tr) if neg_inf_mask else None
        if scale is not None:
            self.functor_kind = "builtin_softmax"
            self._fparams = [scale]
            self._jit_fn = None
            native.load_library() if torch.cuda.is_available() else None
        else:
            self.functor_kind = "lowered"
            self._fparams = []
            fs = functor_lowering.emit_functor(tr, neg_inf_mask=neg_inf_mask, input_ctype=input_ctype)
            self.functor_source = functor_lowering.translation_unit(fs, D, Dv, dtype == torch.bfloat16, sparse=self.sparse_walk)
            # compile now (works without a GPU); loading is deferred to the first call
            native_jit.build(self.functor_source)
            self._jit_fn = None
            # the backward of an elementwise program: source now, compiled when a gradient is first asked for
            if derivative.elementwise_program(tr) and D in (64, 128) and Dv % D == 0:
                self._bwd_source = derivative.backward_translation_unit(derivative.emit_backward_functor(tr), D, dtype == torch.bfloat16)
        self.attention = self._run_parallel

    def _run_parallel(self, q, k, v, *custom, block_mask=None, cache_seqlens=None):
        if self._decode_block is not None:
            run = lambda *ts: self._run_parallel_impl(*ts, block_mask=block_mask, cache_seqlens=cache_seqlens)  # noqa: E731
        else:
            run = self._run_parallel_impl
        if any(t.requires_grad for t in (q, k, v)) and torch.is_grad_enabled():
            if self.has_backward(q, v) and not custom:
                return _SoftmaxAttention.apply(self, q, k, v)
            if self._bwd_source is not None and self._masked_for_backward():
                return _ElementwiseAttention.apply(self, len(custom), q, k, v, *custom)
            return _ForwardOnly.apply(run, q, k, v, *custom)
        return run(q, k, v, *custom)

    def _masked_for_backward(self) -> bool:
        """Masks the backward kernels take: none, causal, bands, and any other mask_mod that does not use the batch or
        head index (as keep bits)."""
        masked = self.mask_kind != native.MASK_NONE or self._sparse_host is not None
        if masked and not self._neg_inf_mask:
            # with another mask value the forward masks nothing element-wise (as the reference: core/lower/lower.py:637-638)
            # while a backward would: refused rather than inconsistent
            return False
        return (self.mask_kind in (native.MASK_NONE, native.MASK_CAUSAL, native.MASK_BAND) and self._decode_block is None and
                (self._sparse_host is None or "bits_q" in self._sparse_host))

    def _mask_bits(self, device):
        """(bits_q, bits_kv) on ``device`` for a general mask_mod, else None."""
        if self._sparse_host is None or "bits_q" not in self._sparse_host:
            return None
        if device not in self._sparse_dev:
            self._sparse_dev[device] = sparse_lowering.to_device(self._sparse_host, device)
        d = self._sparse_dev[device]
        return d["bits_q"], d["bits_kv"], d["tiles_q"], d["tiles_kv"]

    def has_backward(self, q, v) -> bool:
        """Whether gradients flow through this engine for these operands: the built-in softmax (a traced program that
        is softmax attention with a probed scale), no mask, a causal one, a band (sliding windows) or any other mask_mod
        that does not use the batch or head index, dim_qk 128 or 64 and dim_v a multiple of it (the 128 / 256 of the
        reference's suite runs as one backward per 128-column slice of v)."""
        return (self.functor_kind == "builtin_softmax" and self._masked_for_backward() and len(self.final_names) == 1 and
                q.shape[-1] in (64, 128) and v.shape[-1] % q.shape[-1] == 0)

    def _custom_operands(self, custom, B, H, Sq, Skv, device):
        """Checks the custom input tensors against their declared shapes and returns (tensors, element strides over
        (batch, heads, seq_len, seq_len_kv)).  A named axis must have extent 1 (broadcast) or exactly the extent of
        this call, a literal axis its declared extent: the kernel addresses the tensor by strides alone, so anything
        smaller would be read out of bounds."""
        extent = {0: B, 1: H, 2: Sq, 3: Skv}
        names = {0: "batch", 1: "heads", 2: "seq_len", 3: "seq_len_kv"}
        tensors, strides = [], []
        for name, sym, t, want in zip(self.custom_names, self._custom_syms, custom, self._custom_dtypes):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"custom input {name!r} must be a tensor")
            axes = custom_axes(sym)
            if t.dim() != len(axes):
                raise ValueError(f"custom input {name!r}: declared with {len(axes)} axes {tuple(sym.shape_idx)}, got a "
                                 f"tensor of shape {tuple(t.shape)}")
            st = [0, 0, 0, 0]
            for dim, ax in enumerate(axes):
                size = t.shape[dim]
                if ax is None:
                    declared = sym.shape_idx[dim]
                    if declared.isdigit() and size != int(declared):
                        raise ValueError(f"custom input {name!r}: axis {dim} is declared as {declared}, got {size}")
                    if size != 1:
                        raise ValueError(f"custom input {name!r}: axis {dim} ({declared!r}, extent {size}) is not an axis "
                                         "the forward kernel can index; use batch / heads / seq_len / seq_len_kv or 1")
                    continue
                if size != 1 and size != extent[ax]:
                    raise ValueError(f"custom input {name!r}: axis {dim} ({names[ax]}) must have extent 1 or {extent[ax]}, "
                                     f"got {size}")
                if size > 1:
                    st[ax] = t.stride(dim)
            if t.is_cuda and t.device != device:
                raise ValueError(f"custom input {name!r} is on {t.device}, q is on {device}")
            t = t.to(device=device, dtype=want)
            for dim, ax in enumerate(axes):   # strides of the converted tensor
                if ax is not None and t.shape[dim] > 1:
                    st[ax] = t.stride(dim)
            tensors.append(t)
            strides.append(st)
        return tensors, strides

    def _run_parallel_impl(self, q, k, v, *custom, block_mask=None, cache_seqlens=None):
        if len(custom) != len(self.custom_names):
            raise TypeError(f"expected {len(self.custom_names)} custom input tensor(s) {self.custom_names}, got {len(custom)}")
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
            raise ValueError("q, k, v must be [batch, seq, heads, dim]")
        if k.device != q.device or v.device != q.device:
            raise ValueError(f"q, k, v must be on one device (got {q.device}, {k.device}, {v.device})")
        if not q.is_cuda:
            raise native.NativeError("the forward kernel needs CUDA tensors: there is no CPU path")
        B, S, H, _ = q.shape
        tensors, strides = self._custom_operands(custom, B, H, S, k.shape[1], q.device)
        # the entry points launch on the CURRENT device and stream: make q's device current for the whole call
        with torch.cuda.device(q.device):
            sparse = None
            if self._decode_block is not None:
                # block-sparse, variable-length decode (examples/sparse_gqa_decode.py, blockattn_decode_varlen_tl.py):
                # the call's block_mask [B, Hkv, blocks] and cache_seqlens [B] become, on the device, the bitmaps of
                # the KV tiles to visit and the column masks of the tiles kept in part
                sparse = native.decode_tiles(block_mask, cache_seqlens, B, k.shape[2], k.shape[1], self._decode_block, q.device)
            return self._launch_parallel(q, k, v, tensors, strides, sparse)

    def _launch_parallel(self, q, k, v, tensors, strides, sparse=None):
        B, S, H, _ = q.shape
        Dv = v.shape[3]
        o = torch.empty((B, S, H, Dv), dtype=q.dtype, device=q.device)
        finals = [torch.empty((B, H, S), dtype=torch.float32, device=q.device) for _ in self.final_names]
        if sparse is None and self._sparse_host is not None:
            if q.device not in self._sparse_dev:
                self._sparse_dev[q.device] = sparse_lowering.to_device(self._sparse_host, q.device)
            sparse = self._sparse_dev[q.device]
        # split-KV when the launch would leave most SMs idle (decode: few query rows and heads against a long KV): the
        # split results are added up with the weights of the functor's combine (built-in softmax: through the
        # log-sum-exp; lowered functors: the user's OnlineFunc.combine, which needs every split to be non-empty,
        # i.e. no mask)
        splits, workspace = 1, None
        lowered_ok = self.functor_kind == "lowered" and self.mask_kind == native.MASK_NONE
        if sparse is None and Dv <= 128 and q.shape[-1] <= 128 and (self.functor_kind == "builtin_softmax" or lowered_ok):
            splits = self.kv_splits if self.kv_splits is not None else plan_kv_splits(B, H, S, k.shape[1], q.device)
            if splits > 1 and self.functor_kind == "lowered":
                kv_tiles = (k.shape[1] + 127) // 128
                per = -(-kv_tiles // min(splits, kv_tiles))
                splits = -(-kv_tiles // per)          # no split without KV tiles
            if splits > 1:
                workspace = torch.empty(B * splits * H * S * (Dv + native.MAX_ROWSCALES) * 4, dtype=torch.uint8, device=q.device)
        args = native.fill_parallel_args(q, k, v, o, mask_kind=self.mask_kind, mask_band=self.mask_band,
                                         num_splits=splits, workspace=workspace, functor=native.FUNCTOR_SOFTMAX,
                                         fparams=self._fparams, final_rowscales=finals, custom=tensors,
                                         custom_strides=strides, sparse=sparse)
        if self.functor_kind == "builtin_softmax":
            native.parallel_fwd(args)
        else:
            if self._jit_fn is None:
                self._jit_fn = native_jit.load(self.functor_source)
            status = native.device_status_word(q.device.index)
            native.check(self._jit_fn(C.byref(args), native.current_stream_ptr(), status), "attn_b200_parallel_fwd_jit")
        # a lowered functor's combine gives output weights only: its splits' final row scales are not merged
        merged = splits == 1 or self.functor_kind == "builtin_softmax"
        self.last_final_rowscales = dict(zip(self.final_names, finals)) if merged else {}
        return o

    # ------------------------------------------------------------------
    def __call__(self, *args, **kargs):
        if self._decode_block is not None:
            # (q, k, v, *custom tensors, block_mask=..., cache_seqlens=...)
            return self.attention(*args, block_mask=kargs.get("block_mask"), cache_seqlens=kargs.get("cache_seqlens"))
        if kargs.get("block_mask") is not None:
            args = args + (kargs["block_mask"],)
        elif self.block_mask is not None:
            args = args + (self.block_mask,)
        if self.use_varlen:
            args = args + (kargs.get("cache_seqlens"),)
        return self.attention(*args)

    # ------------------------------------------------------------------
    def forward_host(self, q, k, v, *custom, out=None, finals_out=None, batch_chunk=1):
        """Forward pass for q, k, v that live in (pinned) HOST memory: [batch, seq, heads, dim] each.

        The batch is cut into slices of ``batch_chunk`` sequences that travel through three streams — host to
        device, kernel, device to host — so that the copies of neighbouring slices overlap each other (PCIe is full
        duplex) and the kernel.  Returns the output as a pinned host tensor (``out`` if given) and leaves the
        per-row outputs (e.g. ``lse``) in ``finals_out`` / ``self.last_final_rowscales`` as host tensors.  All work is
        ordered after the caller's current stream, and that stream waits for the last copy, so CUDA events recorded
        around the call see all of it.  Custom input tensors are device tensors; one whose leading dimension equals
        the batch is sliced with it.  The reference has no host-side entry; this is the call for a host that keeps
        activations outside the device.
        """
        if q.is_cuda or k.is_cuda or v.is_cuda:
            raise ValueError("forward_host takes host tensors; call the engine itself for device tensors")
        B, S, H, _ = q.shape
        Dv = v.shape[3]
        dev = torch.device("cuda", torch.cuda.current_device())
        if out is None:
            out = torch.empty((B, S, H, Dv), dtype=q.dtype).pin_memory()
        finals_host = {} if finals_out is None else finals_out
        for name in self.final_names:
            if name not in finals_host:
                finals_host[name] = torch.empty((B, H, S), dtype=torch.float32).pin_memory()
        st = getattr(self, "_host_streams", None)
        if st is None or st[0].device != dev:
            st = self._host_streams = tuple(torch.cuda.Stream(device=dev) for _ in range(3))
        s_in, s_run, s_out = st
        cur = torch.cuda.current_stream(dev)
        for s_ in st:
            s_.wait_stream(cur)
        step = max(1, int(batch_chunk))
        for b0 in range(0, B, step):
            b1 = min(B, b0 + step)
            with torch.cuda.stream(s_in):
                dq = q[b0:b1].to(dev, non_blocking=True)
                dk = k[b0:b1].to(dev, non_blocking=True)
                dv = v[b0:b1].to(dev, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(arrived)
                for t in (dq, dk, dv):
                    t.record_stream(s_run)
                cs = [c[b0:b1] if (c.dim() > 0 and c.shape[0] == B and B > 1) else c for c in custom]
                o = self(dq, dk, dv, *cs)
                finals = dict(self.last_final_rowscales)
                done = torch.cuda.Event()
                done.record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                o.record_stream(s_out)
                out[b0:b1].copy_(o, non_blocking=True)
                for name, t in finals.items():
                    t.record_stream(s_out)
                    finals_host[name][b0:b1].copy_(t, non_blocking=True)
        cur.wait_stream(s_out)
        cur.wait_stream(s_run)
        cur.wait_stream(s_in)
        self.last_final_rowscales = finals_host
        return out
