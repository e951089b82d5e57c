"""Symbolic tracing front-end: the objects user-written ``score_mod`` /
``OnlineFunc`` / ``q_mod`` callables operate on.

Behavioural contract (method list, constructor arguments, public attributes)
follows the reference front-end, attention_engine/core/transform/core.py:
``SymbolScalar`` (:35-251), ``SymbolicArray.get_reduce`` (:253-277),
``SymbolicColReduceArray`` (:279-304), ``SymbolicTensor`` (:306-317),
``SymbolicConst`` (:319-328), ``CustomIO`` (:331-349) and the block-mask
helpers (:352-512).  The symbolic autodiff of the reference (:119-199) is not
provided: the native backend is forward-only.

Calling a user function on these objects records a DAG (``prev`` links
between ``SymbolScalar`` objects, ``code`` holding the op node).  The DAG is
consumed by ``core.lower.functor`` which emits a C++ device functor.
"""

from __future__ import annotations

import itertools
from typing import Literal, Optional, Type

import torch
from torch import Tensor

from .graph import *  # noqa: F401,F403  (re-export node classes, as the reference does)
from .graph import (Abs, Add, ColReduceAbsSum, ColReduceMax, ColReduceSum, Const, Div,
                    Exp, Exp2, Log, Log2, Max, MaxBwd, Min, Mul, Neg, Node, ReduceAbsSum,
                    ReduceMax, ReduceSum, Sub, Tanh, Var)

_uid = itertools.count()


class SymbolScalar:
    """A traced value.  ``shape_idx`` names its axes symbolically:
    ``["block_M"]`` is one value per query row, ``["block_M", "block_N"]`` a
    score tile, ``[]`` a constant, anything else a custom-tensor shape."""

    def __init__(self, varname: str, value: Node, prev=None, shape_idx=("block_M",),
                 require_grad: bool = True, dtype: str = "float"):
        self.varname = varname
        self.code = value
        self.prev = list(prev) if prev is not None else []
        self.shape_idx = [str(i) for i in shape_idx]
        self.require_grad = require_grad
        self.dtype = dtype
        self.count = 0
        self.use_list: list[SymbolScalar] = []
        self.allow_reuse = True
        self.lowered = False
        self.visit_count = 0
        self.grad = None
        self.uid = next(_uid)

    # -- bookkeeping kept for source compatibility with reference user code --
    def set_allow_reuse(self, allow_reuse: bool):
        self.allow_reuse = allow_reuse

    def clear_usecount(self):
        self.count = 0
        self.use_list.clear()

    def clear_visit(self):
        self.visit_count = 0
        self.lowered = False

    def clear_codegen(self):
        self.clear_usecount()
        self.clear_visit()

    @property
    def name(self) -> str:
        return self.varname

    @property
    def shape(self):
        return list(self.shape_idx)

    def __repr__(self):
        return f"{type(self).__name__}({self.varname}: {self.code} {self.shape_idx})"

    # -- graph construction --
    def op(self, code: Type[Node], others=None, shape_idx=None, varname_suffix: str | None = None):
        """Record ``code(self, *others)`` and return the new traced value.
        Python numbers among ``others`` become ``SymbolicConst`` leaves."""
        operands = [self]
        for other in (others or []):
            if isinstance(other, bool):
                other = float(other)
            if isinstance(other, (int, float)):
                other = SymbolicConst(other)
            elif isinstance(other, torch.Tensor) and other.numel() == 1:
                other = SymbolicConst(float(other))
            elif not isinstance(other, SymbolScalar):
                raise TypeError(f"unsupported operand {type(other).__name__} in traced expression")
            operands.append(other)
        if shape_idx is None:
            shape_idx = _broadcast_shape(operands)
        stem = self.varname if varname_suffix is None else f"{self.varname}_{varname_suffix}"
        # a [block_M, block_N] result stays a tile object so get_reduce() is available
        tile_cls = next((type(o) for o in operands
                         if isinstance(o, (SymbolicArray, SymbolicColReduceArray))), None)
        out_cls = tile_cls if (tile_cls is not None and len(shape_idx) == 2) else SymbolScalar
        out = out_cls.__new__(out_cls)
        SymbolScalar.__init__(out, f"{stem}_{self.count}", code(*[o.code for o in operands]),
                              operands, shape_idx)
        for o in operands:
            o.use_list.append(out)
            o.count += 1
        return out

    def backward(self, grad=None):
        raise NotImplementedError(
            "symbolic differentiation is not part of the forward-only native backend")

    def _rop(self, code, other):
        return SymbolicConst(other).op(code, [self])

    def __add__(self, other):
        return self.op(Add, [other])

    def __radd__(self, other):
        return self.op(Add, [other])

    def __sub__(self, other):
        return self.op(Sub, [other])

    def __rsub__(self, other):
        return self._rop(Sub, other)

    def __mul__(self, other):
        return self.op(Mul, [other])

    def __rmul__(self, other):
        return self.op(Mul, [other])

    def __truediv__(self, other):
        return self.op(Div, [other])

    def __rtruediv__(self, other):
        return self._rop(Div, other)

    def __neg__(self):
        return self.op(Neg)

    def abs(self):
        return self.op(Abs)

    def tanh(self):
        return self.op(Tanh)

    def exp(self):
        return self.op(Exp)

    def exp2(self):
        return self.op(Exp2)

    def log(self):
        return self.op(Log)

    def log2(self):
        return self.op(Log2)

    def max(self, other):
        return self.op(Max, [other])

    def min(self, other):
        return self.op(Min, [other])

    def maxbwd(self, other1, other2):
        return self.op(MaxBwd, [other1, other2])


def _axis_rank(sym: "SymbolScalar") -> float:
    """How 'wide' a traced value is when broadcast inside the kernel:
    0 constant, 0.5 per-launch scalar tensor, 1 one value per query row, 2 a score tile."""
    if isinstance(sym, SymbolicTensor):
        axes = set(sym.shape_idx)
        if "seq_len_kv" in axes:
            return 1.9
        if "seq_len" in axes:
            return 0.9
        return 0.5
    return float(min(len(sym.shape_idx), 2))


def _broadcast_shape(operands) -> list[str]:
    widest = max(operands, key=_axis_rank)
    rank = _axis_rank(widest)
    if isinstance(widest, SymbolicTensor):
        # a custom tensor broadcast against nothing wider: describe it in tile terms
        return ["block_M", "block_N"] if rank > 1 else (["block_M"] if rank > 0.5 else [])
    return list(widest.shape_idx)


class SymbolicArray(SymbolScalar):
    """A [block_M, block_N] score tile handed to ``OnlineFunc.online_fwd``."""

    def __init__(self, varname: str = "", code: Node | None = None, prev=None,
                 shape_idx=("block_M", "block_N")):
        super().__init__(varname, code if code is not None else Var(" "), prev, shape_idx)

    def get_reduce(self, op: Literal["sum", "max", "abssum"]):
        """Reduce along the last axis (one value per query row)."""
        table = {"sum": ReduceSum, "max": ReduceMax, "abssum": ReduceAbsSum}
        if op not in table:
            raise NotImplementedError(f"row reduction {op!r}")
        return self.op(table[op], shape_idx=self.shape_idx[:-1], varname_suffix=op)


class SymbolicColReduceArray(SymbolScalar):
    """A [num_split, block_M] array for ``OnlineFunc.combine``: reductions run
    over the split axis (the first of the last two)."""

    def __init__(self, varname: str = "", code: Node | None = None, prev=None,
                 shape_idx=("block_M", "block_N")):
        super().__init__(varname, code if code is not None else Var(" "), prev, shape_idx)

    def get_reduce(self, op: Literal["sum", "max", "abssum"]):
        table = {"sum": ColReduceSum, "max": ColReduceMax, "abssum": ColReduceAbsSum}
        if op not in table:
            raise NotImplementedError(f"column reduction {op!r}")
        shape_idx = self.shape_idx[:-2] + [self.shape_idx[-1]]
        return self.op(table[op], shape_idx=shape_idx, varname_suffix=op)


class SymbolicTensor(SymbolScalar):
    """A user-supplied extra kernel input declared through ``CustomIO``."""

    def __init__(self, varname: str, shape: tuple):
        super().__init__(varname, Var(varname), shape_idx=[str(i) for i in shape])


class SymbolicConst(SymbolScalar):
    """A Python number captured at trace time."""

    def __init__(self, value):
        super().__init__(f"float({value})", Const(value), prev=[], shape_idx=[],
                         require_grad=False)


class CustomIO:
    """Declares extra kernel inputs: ``{name: shape}`` where each shape entry
    is an int or one of the symbolic axis names (``"batch"``, ``"heads"``,
    ``"seq_len"``, ``"seq_len_kv"``; the linear pattern adds ``"dimqk"``,
    ``"dimv"``)."""

    def __init__(self, input_tensors: dict[str, tuple] | None = None):
        self.input_tensors: dict[str, SymbolicTensor] = {}
        for k, v in (input_tensors or {}).items():
            self.input_tensors[k] = SymbolicTensor(k, v)

    def __call__(self, tensor_name: str, tensor_shape: tuple):
        if tensor_name in self.input_tensors:
            raise ValueError(f"Tensor {tensor_name} already exists")
        self.input_tensors[tensor_name] = SymbolicTensor(tensor_name, tensor_shape)

        def decorator(func):
            return func
        return decorator


# --------------------------------------------------------------------------
# mask helpers
# --------------------------------------------------------------------------

_DEFAULT_SPARSE_BLOCK_SIZE = 128
BLOCK_SIZE = 128


def _eval_mask_2d(mod_fn, b: int, h: int, q_len: int, kv_len: int, device) -> Tensor:
    """mask_mod evaluated for one (b, h) over the full [q_len, kv_len] grid."""
    bi = torch.tensor(b, device=device)
    hi = torch.tensor(h, device=device)
    q = torch.arange(q_len, device=device).view(-1, 1)
    kv = torch.arange(kv_len, device=device).view(1, -1)
    try:
        out = mod_fn(bi, hi, q, kv)
        out = torch.as_tensor(out, device=device)
        if out.shape != (q_len, kv_len):
            out = out.expand(q_len, kv_len)
        return out.to(torch.bool)
    except Exception:
        fn = mod_fn
        for dims in ((None, None, None, 0), (None, None, 0, None)):
            fn = torch.vmap(fn, in_dims=dims, out_dims=0)
        return fn(bi, hi, q.view(-1), kv.view(-1)).to(torch.bool)


class _Watched(torch.Tensor):
    """A tensor that remembers whether any torch operation was applied to it."""

    touched = False

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        _Watched.touched = True
        plain = lambda x: x.as_subclass(torch.Tensor) if isinstance(x, _Watched) else x  # noqa: E731
        with torch._C.DisableTorchFunctionSubclass():
            return func(*torch.utils._pytree.tree_map(plain, args), **torch.utils._pytree.tree_map(plain, kwargs or {}))


def mask_depends_on_batch_head(mod_fn, B: int, H: int, q_len: int, kv_len: int, device="cpu") -> bool:
    """True when ``mask_mod`` may give different masks for different (batch, head) pairs.

    Decided by use, not by sampling: the mask function is called once with batch and head indices that record
    any operation applied to them.  A function that never touches them cannot depend on them; one that does is
    treated as dependent (the general per-(batch, head) path is always correct).  If the function cannot be
    called on such indices, every (batch, head) pair is compared with the first on a strided sub-grid of positions
    and on the rows and columns next to the diagonal."""
    if B * H <= 1:
        return False
    q = torch.arange(0, q_len, max(1, q_len // 64), device=device).view(-1, 1)
    kv = torch.arange(0, kv_len, max(1, kv_len // 64), device=device).view(1, -1)
    try:
        _Watched.touched = False
        bi = torch.tensor(0, device=device).as_subclass(_Watched)
        hi = torch.tensor(0, device=device).as_subclass(_Watched)
        mod_fn(bi, hi, q, kv)
        return _Watched.touched
    except Exception:
        pass

    def sample(b, h):
        bi = torch.tensor(b, device=device)
        hi = torch.tensor(h, device=device)
        out = torch.as_tensor(mod_fn(bi, hi, q, kv)).to(torch.bool).expand(q.numel(), kv.numel())
        n = min(q_len, kv_len)
        d = torch.arange(n, device=device)
        near = [torch.as_tensor(mod_fn(bi, hi, d, (d + off).clamp(0, kv_len - 1))).to(torch.bool).expand(n) for off in (-1, 0, 1)]
        return torch.cat([out.reshape(-1), *near])

    base = sample(0, 0)
    return any(not torch.equal(base, sample(b, h)) for b in range(B) for h in range(H) if (b, h) != (0, 0))


def create_mask(mod_fn, B: Optional[int], H: Optional[int], Q_LEN: int, KV_LEN: int,
                device: str = "cuda") -> Tensor:
    """Dense bool mask [B, H, Q_LEN, KV_LEN] from a ``mask_mod(b, h, q_idx, kv_idx)``.
    Same result as the reference's vmap construction (core.py:352-398); masks
    that do not depend on (b, h) are evaluated once and expanded (a view), so
    the B*H*S*S tensor is never materialised for them."""
    B = 1 if B is None else B
    H = 1 if H is None else H
    if not mask_depends_on_batch_head(mod_fn, B, H, Q_LEN, KV_LEN, device):
        return _eval_mask_2d(mod_fn, 0, 0, Q_LEN, KV_LEN, device).expand(B, H, Q_LEN, KV_LEN)
    rows = [torch.stack([_eval_mask_2d(mod_fn, b, h, Q_LEN, KV_LEN, device) for h in range(H)])
            for b in range(B)]
    return torch.stack(rows)


def _convert_mask_to_block_mask(mask: Tensor, Q_BLOCK_SIZE=_DEFAULT_SPARSE_BLOCK_SIZE,
                                KV_BLOCK_SIZE=_DEFAULT_SPARSE_BLOCK_SIZE,
                                separate_full_blocks: bool = False):
    """Per-block occupancy of a dense mask: int8 [B, H, ceil(Q/QB), ceil(KV/KVB)],
    1 where any element of the block is kept (core.py:407-453)."""
    assert mask.dtype == torch.bool
    while mask.dim() < 4:
        mask = mask.unsqueeze(0)
    B, H, Q, KV = mask.shape
    nq = -(-Q // Q_BLOCK_SIZE)
    nk = -(-KV // KV_BLOCK_SIZE)
    # work on the distinct (b,h) slices only when the mask is an expanded view
    distinct = mask
    expanded = mask.stride(0) == 0 and mask.stride(1) == 0
    if expanded:
        distinct = mask[:1, :1]
    padded = torch.nn.functional.pad(
        distinct, (0, nk * KV_BLOCK_SIZE - KV, 0, nq * Q_BLOCK_SIZE - Q))
    counts = padded.view(distinct.shape[0], distinct.shape[1], nq, Q_BLOCK_SIZE, nk, KV_BLOCK_SIZE) \
        .sum(dim=(3, 5))
    if expanded:
        counts = counts.expand(B, H, nq, nk)
    if separate_full_blocks:
        full = Q_BLOCK_SIZE * KV_BLOCK_SIZE
        return ((counts > 0) & (counts < full)).to(torch.int8), (counts == full).to(torch.int8)
    return (counts > 0).to(torch.int8), None


def is_causal_mask(mask_tensor: Tensor, block_M: int, block_N: int):
    """True when the block mask [B,H,nq,nk] equals the lower-triangular block
    pattern ``(q+1)*block_M > kv*block_N`` (core.py:455-471)."""
    _, _, M, N = mask_tensor.shape
    q = torch.arange(M, device=mask_tensor.device).view(-1, 1)
    kv = torch.arange(N, device=mask_tensor.device).view(1, -1)
    tri = (q + 1) * block_M > kv * block_N
    return torch.all(mask_tensor.bool() == tri)


def is_less_causal_mask(mask_tensor: Tensor, block_M: int, block_N: int):
    """True when nothing above the block diagonal is kept (core.py:473-488)."""
    _, _, M, N = mask_tensor.shape
    q = torch.arange(M, device=mask_tensor.device).view(-1, 1)
    kv = torch.arange(N, device=mask_tensor.device).view(1, -1)
    upper = (q + 1) * block_M - 1 < kv * block_N
    return torch.all(mask_tensor[..., upper] == 0)


def create_block_mask(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE=None, KV_BLOCK_SIZE=None):
    """int8 block-occupancy mask [B, H, nq, nk] of ``mask_mod`` (core.py:492-506)."""
    Q_BLOCK_SIZE = BLOCK_SIZE if Q_BLOCK_SIZE is None else Q_BLOCK_SIZE
    KV_BLOCK_SIZE = BLOCK_SIZE if KV_BLOCK_SIZE is None else KV_BLOCK_SIZE
    dense = create_mask(mask_mod, B, H, QLen, KVLen, device)
    partial, _ = _convert_mask_to_block_mask(dense, Q_BLOCK_SIZE, KV_BLOCK_SIZE, False)
    return partial


def create_block_idx(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE=None, KV_BLOCK_SIZE=None):
    block_mask = create_block_mask(mask_mod, B, H, QLen, KVLen, device, Q_BLOCK_SIZE, KV_BLOCK_SIZE)
    return torch.nonzero(block_mask, as_tuple=False)
