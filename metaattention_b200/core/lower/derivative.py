"""Backward functor of an elementwise program: the traced ``score_mod`` differentiated in forward mode.

The reference differentiates its DAG symbolically (attention_engine/core/transform/core.py:119-199: every node's
``_backward`` builds gradient nodes, ``MaxBwd`` for the maximum) and lowers the result into its backward template
(core/lower/lower.py:349-436).  Here a program qualifies when nothing but the score tile carries state -- no row
scales, no accumulator rescale, no epilogue (``online_func`` None or the identity; sigmoid and relu attention of the
reference's examples) -- so that P = f(scores) elementwise and

    dV = P^T dO,   dS = dP * f'(scores),   dK = dS^T Q,   dQ = dS K.

``emit_backward_functor`` walks the DAG once and emits, per node, a value and its derivative with respect to the raw
score (dual numbers); the result is the struct the backward kernel template (csrc/attn_bwd.cuh) takes as its functor.
Custom inputs may be fp32 scalars (e.g. the bias of sigmoid attention); tensors with a sequence axis are not covered.
"""

from __future__ import annotations

import math

from core.lower.functor import _f, custom_kind
from core.lower.trace import TracedParallel, init_value

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453


def elementwise_program(tr: TracedParallel) -> bool:
    """True when the traced program is P = f(scores): no row scales, no rescale of the accumulator, no epilogue, no
    final row scales, and only scalar custom inputs."""
    if tr.rowscale_in or tr.rowscale_out or tr.final or tr.o_scale is not None or tr.o_out is not tr.o_in:
        return False
    return all(custom_kind(sym) == "scalar" for sym in tr.custom.values())


class _Dual:
    """Emits `const float vK = ...;` / `const float dK = ...;` statements; a derivative of None is identically zero."""

    def __init__(self):
        self.lines: list[str] = []
        self.count = 0

    def tmp(self, prefix: str, expr: str) -> str:
        self.count += 1
        name = f"{prefix}{self.count}"
        self.lines.append(f"    const float {name} = {expr};")
        return name

    def mul(self, a: str | None, b: str) -> str | None:
        return None if a is None else self.tmp("d", f"{a} * {b}")

    def add(self, a: str | None, b: str | None, sign: str = "+") -> str | None:
        if a is None and b is None:
            return None
        if b is None:
            return a
        if a is None:
            return b if sign == "+" else self.tmp("d", f"-({b})")
        return self.tmp("d", f"{a} {sign} {b}")


def emit_backward_functor(tr: TracedParallel, struct_name: str = "UserBwdFunctor") -> str:
    if not elementwise_program(tr):
        raise NotImplementedError("the backward is derived for elementwise programs only (no row scales, scalar custom inputs)")
    e = _Dual()
    memo: dict[int, tuple[str, str | None]] = {id(tr.scores_in): ("s", "1.0f")}
    for name, sym in tr.index_leaves.items():
        memo[id(sym)] = (f"static_cast<float>({name})", None)
    customs = list(tr.custom.values())
    for k, sym in enumerate(customs):
        memo[id(sym)] = (f"c.cu[{k}]", None)

    def lower(sym):
        key = id(sym)
        if key in memo:
            return memo[key]
        t = sym.code.type
        if t == "Const":
            out = (_f(float(sym.code.value)), None)
        elif t == "Var":
            try:
                out = (_f(init_value(sym.code.name)), None)
            except ValueError:
                raise ValueError(f"free variable {sym.code.name!r} in traced expression is not a kernel input")
        else:
            args = [lower(p) for p in sym.prev]
            if t in ("Add", "Sub"):
                (va, da), (vb, db) = args
                out = (e.tmp("v", f"{va} {'+' if t == 'Add' else '-'} {vb}"), e.add(da, db, "+" if t == "Add" else "-"))
            elif t == "Mul":
                (va, da), (vb, db) = args
                out = (e.tmp("v", f"{va} * {vb}"), e.add(e.mul(da, vb), e.mul(db, va)))
            elif t == "Div":
                (va, da), (vb, db) = args
                v = e.tmp("v", f"{va} / {vb}")
                # (a / b)' = (a' - (a / b) b') / b
                num = e.add(da, e.mul(db, v), "-")
                out = (v, None if num is None else e.tmp("d", f"{num} / {vb}"))
            elif t in ("Max", "Min"):
                (va, da), (vb, db) = args
                v = e.tmp("v", f"{'fmaxf' if t == 'Max' else 'fminf'}({va}, {vb})")
                if da is None and db is None:
                    out = (v, None)
                else:
                    cmp = ">=" if t == "Max" else "<="
                    out = (v, e.tmp("d", f"({va} {cmp} {vb}) ? {da or '0.0f'} : {db or '0.0f'}"))
            elif t == "MaxBwd":
                raise NotImplementedError("MaxBwd appears in gradient graphs only")
            elif t == "Neg":
                ((va, da),) = args
                out = (e.tmp("v", f"-({va})"), None if da is None else e.tmp("d", f"-({da})"))
            elif t == "Abs":
                ((va, da),) = args
                out = (e.tmp("v", f"fabsf({va})"), None if da is None else e.tmp("d", f"({va} >= 0.0f) ? {da} : -({da})"))
            elif t in ("Exp", "Exp2"):
                ((va, da),) = args
                v = e.tmp("v", f"b200::fast_exp2(({va}) * {_f(LOG2E)})" if t == "Exp" else f"b200::fast_exp2({va})")
                out = (v, e.mul(da, v if t == "Exp" else f"({v} * {_f(LN2)})"))
            elif t in ("Log", "Log2"):
                ((va, da),) = args
                v = e.tmp("v", f"b200::fast_log2({va}) * {_f(LN2)}" if t == "Log" else f"b200::fast_log2({va})")
                out = (v, None if da is None else e.tmp("d", f"{da} / ({va}{'' if t == 'Log' else ' * ' + _f(LN2)})"))
            elif t == "Tanh":
                ((va, da),) = args
                v = e.tmp("v", f"b200::fast_tanh({va})")
                out = (v, e.mul(da, f"(1.0f - {v} * {v})"))
            else:
                raise NotImplementedError(f"op {t} has no place in an elementwise program")
        memo[key] = out
        return out

    v, d = lower(tr.scores_out)
    body = "\n".join(e.lines)
    n = max(len(customs), 1)
    loads = "\n".join(f"    c.cu[{k}] = *static_cast<const float*>(p.custom[{k}]);" for k in range(len(customs)))
    return f"""struct {struct_name} {{
  static constexpr bool kUsesStats = false;
  static constexpr bool kNegInfMask = false;
  struct Ctx {{
    float cu[{n}];
  }};
  __device__ static Ctx make(const b200::BwdParams& p) {{
    Ctx c;
    c.cu[0] = 0.0f;
{loads}
    return c;
  }}
  __device__ static void score(float s, float, const Ctx& c, int b, int h, int q_idx, int kv_idx, float& p_out, float& g_out) {{
    (void)b; (void)h; (void)q_idx; (void)kv_idx; (void)c;
{body}
    p_out = {v};
    g_out = {d if d is not None else '0.0f'};
  }}
  __device__ static float grad(float g, float dp, float, const Ctx&) {{ return dp * g; }}
  __device__ static float out_scale(const Ctx&) {{ return 1.0f; }}
}};
"""


def backward_translation_unit(functor_code: str, dim: int, bf16: bool, struct_name: str = "UserBwdFunctor") -> str:
    """Source of a library exporting ``attn_b200_elementwise_bwd_jit`` for one functor, head dim and dtype."""
    b = "true" if bf16 else "false"
    return f"""// generated by core/lower/derivative.py -- do not edit
#include "attn_bwd.cuh"

{functor_code}
extern "C" int attn_b200_elementwise_bwd_jit(const AttnB200ElementwiseBwdArgs* a, void* cuda_stream, int32_t* device_status) {{
  if (a == nullptr || device_status == nullptr) return ATTN_B200_E_INVALID_ARG;
  if (a->dim_qk != {dim} || a->dim_v != {dim} || a->dtype != {1 if bf16 else 0}) return ATTN_B200_E_UNSUPPORTED;
  b200::BwdCall call{{}};
  if (!b200::bwd_mask_of(a->mask_kind, a->mask_left, a->mask_right, a->mask_bits_q, a->mask_bits_kv, a->mask_tiles_q, a->mask_tiles_kv, call)) return ATTN_B200_E_UNSUPPORTED;
  call.q = a->q; call.k = a->k; call.v = a->v; call.d_o = a->d_o;
  call.dq = a->dq; call.dk = a->dk; call.dv = a->dv;
  call.batch = a->batch; call.heads = a->heads; call.heads_kv = a->heads_kv > 0 ? a->heads_kv : a->heads;
  call.seq_q = a->seq_q; call.seq_kv = a->seq_kv; call.dim = a->dim_qk; call.dtype = a->dtype;
  call.scale = 1.0f;
  call.q_stride = a->q_stride; call.k_stride = a->k_stride; call.v_stride = a->v_stride; call.do_stride = a->do_stride;
  call.dq_stride = a->dq_stride; call.dk_stride = a->dk_stride; call.dv_stride = a->dv_stride;
  call.custom = a->custom;
  const int rc = b200::validate_bwd_call(call);
  if (rc != ATTN_B200_OK) return rc;
  return b200::launch_attn_bwd<{struct_name}, {b}, {dim}>(call, static_cast<cudaStream_t>(cuda_stream), device_status);
}}
"""
