"""``LinearAttentionEngine``: chunked linear attention / retention on the native
sm_100a kernel (reference: attention_engine/attn_engine/linear_attn_engine.py:11-65,
lowering core/lower/lower_linear.py:290-409, wrapper linear_tl.py:1240-1268).

``mod(q, k, v, decay, *custom)`` with q ``[B,HQ,T,Dk]``, k ``[B,HK,T,Dk]``,
v ``[B,H,T,Dv]``, decay ``[B,H,T]`` fp32 returns o ``[B,H,T,Dv]``.

The user's ``decay_mod`` / ``k_mod`` / ``v_mod`` are traced once and applied as
whole-tensor torch operations on the device before the kernel, which is what
the reference does with generated PyTorch statements (lower_linear.py:138-206);
``decay_mod`` must produce the natural log of the per-token decay (RetNet:
``decay.log()``).  A ``q_mod`` of the form ``q * const`` is folded into the
kernel (the reference fuses q_mod into its output kernel, linear_tl.py:368-370);
any other ``q_mod`` is applied like the others.  Tuning arguments are accepted
and ignored.
"""

from __future__ import annotations

import ctypes as C

import torch

from core.native import lib as native
from core.transform.core import CustomIO, SymbolicArray, SymbolScalar
from core.transform.graph import Var


def _align(a, b):
    """Broadcast rule of the reference's whole-tensor statements (codegen/tl_gen.py:253-262):
    operands are aligned on their LEADING axes; the shorter one gets trailing singleton axes."""
    if isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.dim() != b.dim():
        if a.dim() < b.dim():
            a = a.reshape(a.shape + (1,) * (b.dim() - a.dim()))
        else:
            b = b.reshape(b.shape + (1,) * (a.dim() - b.dim()))
    return a, b


def eval_tensor_expr(sym: SymbolScalar, env: dict, memo: dict | None = None):
    """Evaluate a traced whole-tensor expression with torch (on whatever device the leaves live)."""
    memo = {} if memo is None else memo
    key = id(sym)
    if key in memo:
        return memo[key]
    if key in env:
        return env[key]
    t = sym.code.type
    if t == "Const":
        val = float(sym.code.value)
    elif t == "Var":
        raise ValueError(f"free variable {sym.code.name!r} in a linear-attention mod")
    else:
        a = [eval_tensor_expr(p, env, memo) for p in sym.prev]
        if len(a) == 2:
            a = list(_align(a[0], a[1]))
        as_t = lambda x: x if isinstance(x, torch.Tensor) else torch.tensor(x)  # noqa: E731
        if t == "Add":
            val = a[0] + a[1]
        elif t == "Sub":
            val = a[0] - a[1]
        elif t == "Mul":
            val = a[0] * a[1]
        elif t == "Div":
            val = a[0] / a[1]
        elif t == "Neg":
            val = -a[0]
        elif t == "Abs":
            val = torch.abs(as_t(a[0]))
        elif t == "Exp":
            val = torch.exp(as_t(a[0]))
        elif t == "Exp2":
            val = torch.exp2(as_t(a[0]))
        elif t == "Log":
            val = torch.log(as_t(a[0]))
        elif t == "Log2":
            val = torch.log2(as_t(a[0]))
        elif t == "Tanh":
            val = torch.tanh(as_t(a[0]))
        elif t == "Max":
            val = torch.maximum(*[x if isinstance(x, torch.Tensor) else torch.tensor(x, device=as_t(a[0]).device if isinstance(a[0], torch.Tensor) else a[1].device, dtype=torch.float32) for x in a])
        else:
            raise NotImplementedError(f"op {t} in a linear-attention mod")
    memo[key] = val
    return val


def _depends_on(sym: SymbolScalar, leaf: SymbolScalar) -> bool:
    return sym is leaf or any(_depends_on(p, leaf) for p in sym.prev)


def _constant_multiple(out: SymbolScalar, leaf: SymbolScalar):
    """If ``out`` is ``leaf * c`` (or ``c * leaf``, ``leaf / c``) for a Python constant c, return c."""
    if out is leaf:
        return 1.0
    if out.code.type in ("Mul", "Div") and len(out.prev) == 2:
        a, b = out.prev
        if a is leaf and b.code.type == "Const":
            c = float(b.code.value)
            return c if out.code.type == "Mul" else 1.0 / c
        if out.code.type == "Mul" and b is leaf and a.code.type == "Const":
            return float(a.code.value)
    return None


def _column_range_ld(t) -> int:
    """The row pitch of t [B, H, T, w] if it is a column range of a contiguous [B, H, T, ld] tensor that the kernel can
    read in place (16-byte aligned start, ld a multiple of 8), else 0."""
    B, H, T, w = t.shape
    ld = t.stride(2)
    if (t.stride(3) == 1 and ld > w and ld % 8 == 0 and t.stride(1) == T * ld and t.stride(0) == H * T * ld
            and t.data_ptr() % 16 == 0):
        return ld
    return 0


def linear_attention_forward(q, k, v, log_decay, q_scale: float = 1.0, normalize: bool = False, eps: float = 1e-5,
                             out_dtype=None, v_scale=None, precise: bool = False):
    """q,k: [B,H,T,Dk]; v: [B,H,T,Dv] (fp16/bf16 CUDA); log_decay: [B,H,T] fp32, natural log of the
    per-token decay.  Returns o [B,H,T,Dv] in the input dtype, or in fp32 with ``out_dtype=torch.float32``
    (the kernel's accumulators without the output rounding).  ``normalize`` applies a per-(batch, head,
    token) normalisation over Dv (zero mean, unit variance, no affine) to the output.  ``v_scale`` [B,H,T] (fp32) is a
    per-token factor on the rows of v, applied inside the kernel.  ``precise``: the decayed scores of a block keep a
    16-bit remainder beside their 16-bit value (a second P V pass)."""
    if out_dtype not in (None, q.dtype, torch.float32):
        raise native.NativeError("out_dtype must be the input dtype or torch.float32")
    f32_out = out_dtype == torch.float32
    if not q.is_cuda:
        raise native.NativeError("linear attention needs CUDA tensors")
    if q.dtype not in native.DTYPE_CODES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise native.NativeError("q, k, v must share dtype float16 or bfloat16")
    B, _, T, Dk = q.shape
    H = v.shape[1]
    if H % q.shape[1] != 0 or H % k.shape[1] != 0:
        raise native.NativeError("the heads of v must be a multiple of the heads of q and of k")
    Dv = v.shape[-1]
    if Dv % 128 != 0:
        # the kernel works on 128-column slices of dim_v: a narrower v (Mamba2's head dim 64) is padded with
        # zero columns, which stay zero in the output and are cut off again
        if normalize:
            raise native.NativeError("normalize needs dim_v to be a multiple of 128")
        pad = 128 - Dv % 128
        o = linear_attention_forward(q, k, torch.nn.functional.pad(v, (0, pad)), log_decay, q_scale, False, eps, out_dtype, v_scale,
                                     precise)
        return o[..., :Dv].contiguous()
    # q and k may be column ranges of wider contiguous tensors (the backward's contractions over ranges of dim_v)
    q_ld, k_ld = _column_range_ld(q), _column_range_ld(k)
    q = q if q_ld else q.contiguous()
    k = k if k_ld else k.contiguous()
    v = v.contiguous()
    log_decay = log_decay.to(dtype=torch.float32, device=q.device).expand(B, H, T).contiguous()
    if v_scale is not None:
        v_scale = v_scale.to(dtype=torch.float32, device=q.device).expand(B, H, T).contiguous()
    with torch.cuda.device(q.device):
        o = torch.empty((B, H, T, Dv), dtype=torch.float32 if f32_out else q.dtype, device=q.device)
        a = native.LinearArgs()
        a.dtype_out = native.DTYPE_OUT_FP32 if f32_out else native.DTYPE_OUT_SAME
        a.q, a.k, a.v, a.log_decay, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), log_decay.data_ptr(), o.data_ptr()
        a.v_scale = v_scale.data_ptr() if v_scale is not None else None
        a.batch, a.heads, a.seq, a.dim_qk, a.dim_v = B, H, T, Dk, Dv
        a.heads_q, a.heads_k = q.shape[1], k.shape[1]
        a.q_ld, a.k_ld = q_ld, k_ld
        a.dtype = native.DTYPE_CODES[q.dtype]
        a.normalize = 1 if normalize else 0
        a.precise = 1 if precise else 0
        a.q_scale = float(q_scale)
        a.norm_eps = float(eps)
        lib = native.load_library()
        need = int(lib.attn_b200_linear_workspace_bytes(C.byref(a)))
        ws = None
        if need > 0:
            ws = torch.empty(need, dtype=torch.uint8, device=q.device)
            a.workspace, a.workspace_bytes = ws.data_ptr(), need
        native.check(lib.attn_b200_linear_fwd(C.byref(a), native.current_stream_ptr()), "attn_b200_linear_fwd")
    return o


def _rows(t, col0=0, width=None, reverse=False):
    """Columns [col0, col0 + width) of t [B, H, T, cols], time reversed if asked, contiguous: one pass of the library's
    row-gather kernel (torch.flip alone runs at a fifth of the copy rate)."""
    width = t.shape[-1] - col0 if width is None else width
    if not reverse:
        return t[..., col0:col0 + width]    # read in place by the kernel (a pitch instead of a copy)
    if width % 8 == 0 and col0 % 8 == 0 and t.shape[-1] % 8 == 0:
        return native.rows_copy(t, col0, width, reverse)
    part = t[..., col0:col0 + width]
    return (part.flip(2) if reverse else part).contiguous()


def _sum_cast(parts, dtype, reverse=False):
    """Sum of the fp32 partial results, rounded to ``dtype``, time reversed if asked: one pass for up to two parts."""
    while len(parts) > 2:
        parts = [parts[0] + parts[1]] + parts[2:]
    if parts[0].shape[-1] % 8 == 0:
        return native.rows_sum_cast(parts[0], parts[1] if len(parts) > 1 else None, dtype, reverse)
    out = (parts[0] + parts[1] if len(parts) > 1 else parts[0]).to(dtype)
    return out.flip(2) if reverse else out


def _retention_parts(qc, kc, vc, log_decay, q_scale, precise=False):
    """o_i = q_scale * sum_{j<=i} exp(G_i - G_j) (qc_i . kc_j) vc_j on the forward kernel with fp32 output, for any width
    of the contraction, as a list of partial results to be added: the sum is linear in the scores, so a contraction
    wider than the kernel's 256 columns is the sum over column ranges it does cover (widths 256 / 128 / 64, the last one
    zero-padded).  The kernel reads the column ranges of qc and kc in place."""
    D = qc.shape[-1]
    parts, start = [], 0
    while start < D:
        width = next((w for w in (256, 128, 64) if D - start >= w), 64)
        have = min(width, D - start)
        qs, ks = _rows(qc, start, have), _rows(kc, start, have)
        if have < width:
            qs, ks = torch.nn.functional.pad(qs, (0, width - have)), torch.nn.functional.pad(ks, (0, width - have))
        parts.append(linear_attention_forward(qs, ks, vc, log_decay, q_scale, out_dtype=torch.float32, precise=precise))
        start += width
    return parts


def linear_attention_backward(q, k, v, log_decay, d_o, q_scale: float = 1.0, need_dg: bool = False):
    """(dq, dk, dv[, dg]) of ``linear_attention_forward`` (no normalisation), the job of the reference's three backward
    kernels (core/template/tl_template/linear/linear_tl.py:461-975), as five runs of the forward kernel.  With
    D_ij = exp(G_i - G_j) for j <= i:

        dq_i = q_scale * sum_{j<=i} D_ij (do_i . v_j) k_j      = retention(q = do, k = v, v = k)
        dv_j = q_scale * sum_{i>=j} D_ij (q_i . k_j) do_i      = retention(q = k, k = q, v = do) with time reversed
        dk_j = q_scale * sum_{i>=j} D_ij (do_i . v_j) q_i      = retention(q = v, k = do, v = q) with time reversed

    Reversing time turns the anti-causal sums into causal ones; position u of the reversed sequence then carries the
    log-decay of token T - u (0 for u = 0), so that the reversed cumulative sums reproduce the same D_ij.  The two
    contractions over dim_v go through ``_retention_parts`` (dim_v may exceed the kernel's 256 columns of dim_qk).
    Reversals, column ranges and the sums of the partial results are single passes of the library's row kernels.

    ``need_dg``: also the gradient with respect to the per-token log-decay, fp32 [B, H, T].  A score A_ij depends on the
    log-decays of tokens j+1..i, so dg_t = sum_{i>=t, j<t} dA_ij A_ij; with dG_i = q_i . dq_i - k_i . dk_i (row sums
    minus column sums of dA o A) that is the reversed cumulative sum of dG — what the reference's dqkg kernel and its
    ``compute_final_dg`` produce per chunk (linear_tl.py:63-76, 638-814).  dg is a difference of sums over dq and dk:
    those runs then keep the 16-bit remainder of their decayed scores."""
    d_o = d_o.to(q.dtype)
    B, H, T, _ = q.shape
    ld = log_decay.to(dtype=torch.float32, device=q.device).expand(B, H, T)
    ld_rev = torch.cat([torch.zeros_like(ld[..., :1]), ld.flip(-1)[..., :-1]], dim=-1).contiguous()
    dq_parts = _retention_parts(d_o, v, k, ld, q_scale, precise=need_dg)
    dq = _sum_cast(dq_parts, q.dtype)
    qr, kr, dr = _rows(q, reverse=True), _rows(k, reverse=True), _rows(d_o, reverse=True)
    # dv: dim_qk fits the kernel, so it is one run that leaves the kernel in the operands' dtype
    dv = _rows(linear_attention_forward(kr, qr, dr, ld_rev, q_scale), reverse=True)
    # dk contracts over column ranges of the reversed v and dO: dO is reversed already (whole, for dv) and v is reversed
    # once; the kernel reads the ranges in place
    dk_parts = _retention_parts(_rows(v, reverse=True), dr, qr, ld_rev, q_scale, precise=need_dg)
    dk = _sum_cast(dk_parts, k.dtype, reverse=True)
    if not need_dg:
        return dq, dk, dv
    dq32 = sum(dq_parts[1:], dq_parts[0])
    dk32_rev = sum(dk_parts[1:], dk_parts[0])
    d_cum = (q.float() * dq32).sum(-1) - (kr.float() * dk32_rev).sum(-1).flip(-1)
    dg = d_cum.flip(-1).cumsum(-1).flip(-1)
    return dq, dk, dv, dg


class _ForwardOnly(torch.autograd.Function):
    @staticmethod
    def forward(ctx, runner, *tensors):
        return runner(*[t.detach() for t in tensors])

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("the B200-native backend differentiates linear attention only without output "
                                  "normalisation")


class _LinearAttention(torch.autograd.Function):
    """Chunked linear attention of operands that have been through their mods, with its backward
    (``linear_attention_backward``): the counterpart of the kernels inside the reference's ``LinearAttention`` autograd
    function (core/template/tl_template/linear/linear_tl.py:1237-1333).  The reference differentiates the mods with
    generated statements (``*_mod_bwd_expr``, :1322-1329); here they are torch operations in front of this function and
    torch's autograd carries dq, dk, dv and the log-decay's gradient through them, custom inputs included."""

    @staticmethod
    def forward(ctx, q, k, v, log_decay, q_scale):
        o = linear_attention_forward(q.detach(), k.detach(), v.detach(), log_decay.detach(), q_scale=q_scale)
        ctx.save_for_backward(q, k, v, log_decay)
        ctx.q_scale = q_scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, log_decay = ctx.saved_tensors
        B, H, T, _ = v.shape
        hq, hk = q.shape[1], k.shape[1]
        qe = q.repeat_interleave(H // hq, dim=1) if hq != H else q
        ke = k.repeat_interleave(H // hk, dim=1) if hk != H else k
        need_dg = ctx.needs_input_grad[3]
        res = linear_attention_backward(qe, ke, v, log_decay, d_o, ctx.q_scale, need_dg=need_dg)
        dq, dk, dv = res[:3]
        if hq != H:   # heads that shared one q head: their gradients add up
            dq = dq.view(B, hq, H // hq, T, -1).float().sum(2).to(dq.dtype)
        if hk != H:
            dk = dk.view(B, hk, H // hk, T, -1).float().sum(2).to(dk.dtype)
        dg = res[3].sum_to_size(log_decay.shape).to(log_decay.dtype) if need_dg else None
        return dq, dk, dv, dg, None


class LinearAttentionEngine:
    def __init__(self, qkv_meta, q_mod=None, k_mod=None, v_mod=None, decay_mod=None, custom_io=None,
                 tune=False, tune_filename="tune_result", tune_bwd=False):
        self.qkv_meta = qkv_meta
        self.custom_io = custom_io if custom_io is not None else CustomIO()
        self.custom_names = list(self.custom_io.input_tensors.keys())
        self.normalize_output = False
        B, HQ, T, Dk = qkv_meta[0].shape
        self.HK = qkv_meta[1].shape[1]
        self.H = qkv_meta[2].shape[1]
        self.Dv = qkv_meta[2].shape[3]
        if Dk not in (64, 128, 256):
            raise NotImplementedError(f"linear attention kernel covers dim_qk in (64,128,256) (got {Dk})")
        if self.H % HQ != 0 or self.H % self.HK != 0:
            raise NotImplementedError(f"v heads ({self.H}) must be a multiple of q heads ({HQ}) and k heads ({self.HK})")
        # trace the mods once
        self._leaves = {
            "q": SymbolicArray("q", Var("q"), shape_idx=["B", "H", "T", "D"]),
            "k": SymbolicArray("k", Var("k"), shape_idx=["B", "H", "T", "D"]),
            "v": SymbolicArray("v", Var("v"), shape_idx=["B", "H", "T", "D"]),
            "decay": SymbolicArray("decay", Var("decay"), shape_idx=["B", "H", "T"]),
        }
        self._mods = {}
        for name, fn in (("q", q_mod), ("k", k_mod), ("v", v_mod), ("decay", decay_mod)):
            self._mods[name] = fn(self._leaves[name], self.custom_io) if fn is not None else None
        self.q_scale = 1.0
        if self._mods["q"] is not None:
            c = _constant_multiple(self._mods["q"], self._leaves["q"])
            if c is not None:
                self.q_scale = c
                self._mods["q"] = None
        # v_mod = v * t with t free of v (Mamba2: v * dt[batch, heads, seq_len]): the factor goes into the kernel, which
        # rescales the rows of v anyway, instead of a whole-tensor multiply before it (the fused v_mod of the
        # reference, core/lower/lower_linear.py:211-287)
        self._v_scale_expr = None
        vm = self._mods["v"]
        if vm is not None and vm.code.type == "Mul" and len(vm.prev) == 2:
            a, b = vm.prev
            other = b if a is self._leaves["v"] else a if b is self._leaves["v"] else None
            if other is not None and not _depends_on(other, self._leaves["v"]):
                self._v_scale_expr = other
                self._mods["v"] = None
        self.attention = self._run

    def _apply(self, name, tensor, custom_env):
        out = self._mods[name]
        if out is None:
            return tensor
        env = dict(custom_env)
        env[id(self._leaves[name])] = tensor.float()
        res = eval_tensor_expr(out, env)
        return res if name == "decay" else res.to(tensor.dtype)

    def has_backward(self) -> bool:
        """Gradients flow to q, k, v, the decay and the custom inputs, through every mod, unless the output is
        normalised."""
        return not self.normalize_output

    def _run(self, q, k, v, decay, *custom):
        tensors = [t for t in (q, k, v, decay) + tuple(custom) if isinstance(t, torch.Tensor)]
        if torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
            if self.has_backward():
                return self._run_differentiable(q, k, v, decay, *custom)
            return _ForwardOnly.apply(self._run_impl, q, k, v, decay, *custom)
        return self._run_impl(q, k, v, decay, *custom)

    def _run_differentiable(self, q, k, v, decay, *custom):
        """The mods as torch operations that autograd records (a factor on v that the forward-only path hands to the
        kernel is an explicit multiply here), then the kernel with its backward."""
        if len(custom) != len(self.custom_names):
            raise TypeError(f"expected custom tensors {self.custom_names}")
        cenv = {id(self.custom_io.input_tensors[n]): t.float() for n, t in zip(self.custom_names, custom)}
        q = self._apply("q", q, cenv)
        k = self._apply("k", k, cenv)
        v = self._apply("v", v, cenv)
        if self._v_scale_expr is not None:
            t = eval_tensor_expr(self._v_scale_expr, cenv)
            t = t if isinstance(t, torch.Tensor) else torch.tensor(float(t), device=v.device)
            f, g = _align(v.float(), t)
            v = (f * g).to(v.dtype)
        log_decay = self._apply("decay", decay.float(), cenv)
        return _LinearAttention.apply(q, k, v, log_decay, self.q_scale)

    def _run_impl(self, q, k, v, decay, *custom):
        if len(custom) != len(self.custom_names):
            raise TypeError(f"expected custom tensors {self.custom_names}")
        cenv = {id(self.custom_io.input_tensors[n]): t.float() for n, t in zip(self.custom_names, custom)}
        q = self._apply("q", q, cenv)
        k = self._apply("k", k, cenv)
        v = self._apply("v", v, cenv)
        v_scale = None
        if self._v_scale_expr is not None:
            t = eval_tensor_expr(self._v_scale_expr, cenv)
            t = t if isinstance(t, torch.Tensor) else torch.tensor(float(t), device=v.device)
            if t.dim() <= 3 and (t.dim() < 3 or t.shape[-1] in (1, v.shape[2])):
                v_scale = t.reshape(t.shape + (1,) * (3 - t.dim())) if t.dim() < 3 else t   # leading axes: batch, heads, token
            else:   # a factor with a feature axis: no per-token scalar, multiply before the kernel
                f, g = _align(v.float(), t)
                v = (f * g).to(v.dtype)
        log_decay = self._apply("decay", decay.float(), cenv)
        B, _, T, _ = q.shape
        H = v.shape[1]
        # fewer q / k heads than v heads: each group serves H / HQ consecutive heads (the grouping of the
        # Mamba2 reference, testing/test.py:222,271); the kernel reads the shared head, nothing is replicated
        return linear_attention_forward(q, k, v, log_decay, q_scale=self.q_scale, normalize=self.normalize_output, v_scale=v_scale)

    def __call__(self, *args, **kargs):
        return self.attention(*args, **kargs)
