"""Lowering of a traced parallel-pattern DAG into the source of a C++ device
functor for the sm_100a forward kernel (csrc/parallel_fwd.cuh).

This replaces the reference's DAG -> TileLang / CuTe text emitters
(attention_engine/core/codegen/tl_gen.py:7-132, :135-233, :306-370).  The op
vocabulary is the same (core/transform/graph.py OP_TABLE); conventions kept:
``Exp`` is evaluated as exp2(x * log2 e) and ``Log`` as log2(x) * ln 2
(tl_gen.py:89-108), ``Tanh`` uses the hardware approximation (tl_gen.py:113-117),
Python numbers become constants, a "-inf" initial row scale becomes -1e38
(core/lower/lower.py:24-30).

In the kernel one thread owns one query row: a [block_M, block_N] tile value
is a register array of N floats, a per-row value is a scalar.  While walking
the DAG a tile value is kept in the lazy form ``alpha * x[i] + beta`` with
row-level ``alpha`` / ``beta``; chains of additions and multiplications by
row values or constants therefore collapse into one FMA per element in front
of the next transcendental (softmax becomes FFMA + EX2 per element, the tanh
form of sigmoid FFMA + TANH + FFMA).
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass

from core.lower.trace import TracedParallel, custom_axes

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453


def _f(x: float) -> str:
    """C++ float literal."""
    if math.isinf(x):
        return "INFINITY" if x > 0 else "(-INFINITY)"
    if math.isnan(x):
        raise ValueError("NaN constant in traced expression")
    r = repr(float(x))
    if "e" not in r and "." not in r:
        r += ".0"
    return r + "f"


@dataclass
class Const:
    value: float


@dataclass
class Row:
    expr: str  # name of a float variable (or a parenthesised expression) valid at row scope


@dataclass
class Tile:
    name: str                  # float array of kN elements
    alpha: object = None       # None (=1) | Const | Row
    beta: object = None        # None (=0) | Const | Row


class _Body:
    """Accumulates the statements of one functor method."""

    def __init__(self, n_sym: str):
        self.lines: list[str] = []
        self.count = 0
        self.n = n_sym

    def fresh(self, prefix: str) -> str:
        self.count += 1
        return f"{prefix}{self.count}"

    def stmt(self, line: str):
        self.lines.append(line)

    def loop(self, body: str):
        self.lines.append("#pragma unroll")
        self.lines.append(f"for (int i = 0; i < {self.n}; ++i) {{ {body} }}")

    # ---- row-level arithmetic (constants folded) ----
    def rexpr(self, v) -> str:
        return _f(v.value) if isinstance(v, Const) else v.expr

    def rnew(self, expr: str) -> Row:
        name = self.fresh("r")
        self.stmt(f"const float {name} = {expr};")
        return Row(name)

    def rbin(self, op: str, a, b):
        if isinstance(a, Const) and isinstance(b, Const):
            x, y = a.value, b.value
            if op == "Add":
                return Const(x + y)
            if op == "Sub":
                return Const(x - y)
            if op == "Mul":
                return Const(x * y)
            if op == "Div":
                return Const(x / y)
            if op == "Max":
                return Const(max(x, y))
            if op == "Min":
                return Const(min(x, y))
        # identities that keep generated code small
        if op == "Mul":
            for u, w in ((a, b), (b, a)):
                if isinstance(u, Const) and u.value == 1.0:
                    return w
                if isinstance(u, Const) and u.value == 0.0:
                    return Const(0.0)
        if op == "Add":
            for u, w in ((a, b), (b, a)):
                if isinstance(u, Const) and u.value == 0.0:
                    return w
        if op == "Sub" and isinstance(b, Const) and b.value == 0.0:
            return a
        ea, eb = self.rexpr(a), self.rexpr(b)
        fmt = {"Add": "{0} + {1}", "Sub": "{0} - {1}", "Mul": "{0} * {1}", "Div": "{0} / {1}",
               "Max": "fmaxf({0}, {1})", "Min": "fminf({0}, {1})"}[op]
        return self.rnew(fmt.format(ea, eb))

    def runary(self, op: str, a):
        if isinstance(a, Const):
            x = a.value
            try:
                table = {"Neg": lambda: -x, "Abs": lambda: abs(x), "Exp": lambda: math.exp(x),
                         "Exp2": lambda: 2.0 ** x, "Log": lambda: math.log(x), "Log2": lambda: math.log2(x),
                         "Tanh": lambda: math.tanh(x)}
                return Const(table[op]())
            except (ValueError, OverflowError):
                pass
        e = self.rexpr(a)
        fmt = {"Neg": "-({0})", "Abs": "fabsf({0})",
               "Exp": f"b200::fast_exp2(({{0}}) * {_f(LOG2E)})", "Exp2": "b200::fast_exp2({0})",
               "Log": f"b200::fast_log2({{0}}) * {_f(LN2)}", "Log2": "b200::fast_log2({0})",
               "Tanh": "b200::fast_tanh({0})"}[op]
        return self.rnew(fmt.format(e))

    # ---- tile helpers ----
    def elem(self, t: Tile) -> str:
        """Expression of element i of a lazy tile."""
        x = f"{t.name}[i]"
        if t.alpha is None and t.beta is None:
            return x
        if t.alpha is None:
            return f"({x} + {self.rexpr(t.beta)})"
        if t.beta is None:
            return f"({x} * {self.rexpr(t.alpha)})"
        return f"fmaf({x}, {self.rexpr(t.alpha)}, {self.rexpr(t.beta)})"

    def materialize(self, t: Tile) -> Tile:
        if t.alpha is None and t.beta is None:
            return t
        name = self.fresh("t")
        self.stmt(f"float {name}[{self.n}];")
        self.loop(f"{name}[i] = {self.elem(t)};")
        return Tile(name)

    def tile_map(self, expr_of_elems: str, *tiles: Tile) -> Tile:
        """New tile whose element i is ``expr_of_elems`` formatted with the element expressions."""
        name = self.fresh("t")
        self.stmt(f"float {name}[{self.n}];")
        self.loop(f"{name}[i] = {expr_of_elems.format(*[self.elem(t) for t in tiles])};")
        return Tile(name)


class _Lowerer:
    def __init__(self, body: _Body, leaves: dict):
        self.b = body
        self.memo: dict[int, object] = dict(leaves)

    def alpha(self, t: Tile):
        return t.alpha if t.alpha is not None else Const(1.0)

    def beta(self, t: Tile):
        return t.beta if t.beta is not None else Const(0.0)

    @staticmethod
    def _norm(v):
        return v

    def mk(self, name, alpha, beta) -> Tile:
        if isinstance(alpha, Const) and alpha.value == 1.0:
            alpha = None
        if isinstance(beta, Const) and beta.value == 0.0:
            beta = None
        return Tile(name, alpha, beta)

    def lower(self, sym):
        key = id(sym)
        if key in self.memo:
            return self.memo[key]
        val = self._lower(sym)
        self.memo[key] = val
        return val

    def _lower(self, sym):
        b = self.b
        t = sym.code.type
        if t == "Const":
            return Const(float(sym.code.value))
        if t == "Var":
            from core.lower.trace import init_value
            try:
                return Const(init_value(sym.code.name))
            except ValueError:
                raise ValueError(f"free variable {sym.code.name!r} in traced expression is not a kernel input")
        args = [self.lower(p) for p in sym.prev]
        if t in ("Add", "Sub", "Mul", "Div", "Max", "Min"):
            x, y = args
            xt, yt = isinstance(x, Tile), isinstance(y, Tile)
            if not xt and not yt:
                return b.rbin(t, x, y)
            if xt and yt:
                fmt = {"Add": "{0} + {1}", "Sub": "{0} - {1}", "Mul": "{0} * {1}", "Div": "{0} / {1}",
                       "Max": "fmaxf({0}, {1})", "Min": "fminf({0}, {1})"}[t]
                return b.tile_map(fmt, x, y)
            if xt:  # tile (op) row
                if t == "Add":
                    return self.mk(x.name, x.alpha, b.rbin("Add", self.beta(x), y))
                if t == "Sub":
                    return self.mk(x.name, x.alpha, b.rbin("Sub", self.beta(x), y))
                if t == "Mul":
                    return self.mk(x.name, b.rbin("Mul", self.alpha(x), y), b.rbin("Mul", self.beta(x), y))
                if t == "Div":
                    inv = b.rbin("Div", Const(1.0), y)
                    return self.mk(x.name, b.rbin("Mul", self.alpha(x), inv), b.rbin("Mul", self.beta(x), inv))
                fn = "fmaxf" if t == "Max" else "fminf"
                return b.tile_map(fn + "({0}, " + b.rexpr(y) + ")", x)
            # row (op) tile
            if t == "Add":
                return self.mk(y.name, y.alpha, b.rbin("Add", x, self.beta(y)))
            if t == "Sub":
                return self.mk(y.name, b.runary("Neg", self.alpha(y)), b.rbin("Sub", x, self.beta(y)))
            if t == "Mul":
                return self.mk(y.name, b.rbin("Mul", x, self.alpha(y)), b.rbin("Mul", x, self.beta(y)))
            if t == "Div":
                return b.tile_map(b.rexpr(x) + " / {0}", y)
            fn = "fmaxf" if t == "Max" else "fminf"
            return b.tile_map(fn + "(" + b.rexpr(x) + ", {0})", y)
        if t in ("Neg", "Abs", "Exp", "Exp2", "Log", "Log2", "Tanh"):
            (x,) = args
            if not isinstance(x, Tile):
                return b.runary(t, x)
            if t == "Neg":
                return self.mk(x.name, b.runary("Neg", self.alpha(x)), b.runary("Neg", self.beta(x)))
            if t == "Exp":
                # exp(a*x+b) = exp2(a*log2e*x + b*log2e): the base change is folded into the FMA
                x2 = self.mk(x.name, b.rbin("Mul", self.alpha(x), Const(LOG2E)), b.rbin("Mul", self.beta(x), Const(LOG2E)))
                return b.tile_map("b200::fast_exp2({0})", x2)
            if t == "Exp2":
                return b.tile_map("b200::fast_exp2({0})", x)
            if t == "Log":
                return self.mk(b.tile_map("b200::fast_log2({0})", x).name, Const(LN2), None)
            if t == "Log2":
                return b.tile_map("b200::fast_log2({0})", x)
            if t == "Tanh":
                return b.tile_map("b200::fast_tanh({0})", x)
            return b.tile_map("fabsf({0})", x)
        if t in ("ReduceSum", "ReduceMax", "ReduceAbsSum"):
            (x,) = args
            if not isinstance(x, Tile):
                raise ValueError(f"{t} applied to a value that is not a score tile")
            if t == "ReduceMax" and isinstance(self.alpha(x), Const) and self.alpha(x).value > 0:
                # max(a*x+b) = a*max(x)+b for a constant a > 0: reduce the raw values
                acc = self._reduce(Tile(x.name), "fmaxf({0}, {1})", None)
                return b.rbin("Add", b.rbin("Mul", acc, self.alpha(x)), self.beta(x))
            if t == "ReduceMax":
                return self._reduce(x, "fmaxf({0}, {1})", None)
            if t == "ReduceSum":
                return self._reduce(x, "{0} + {1}", "0.0f")
            return self._reduce(x, "{0} + fabsf({1})", "0.0f")
        raise NotImplementedError(f"op {t} is not supported by the functor emitter")

    def _reduce(self, x: Tile, combine: str, init: str | None) -> Row:
        """Four independent partial accumulators, combined at the end."""
        b = self.b
        base = b.fresh("a")
        e = b.elem(x)
        parts = [f"{base}_{k}" for k in range(4)]
        if init is None:  # max: start from the first four elements
            for k in range(4):
                b.stmt(f"float {parts[k]} = {e.replace('[i]', f'[{k}]')};")
            start = 4
        else:
            for k in range(4):
                b.stmt(f"float {parts[k]} = {init};")
            start = 0
        b.stmt("#pragma unroll")
        b.stmt(f"for (int i = {start}; i < {b.n}; ++i) {{ float& acc = (i & 3) == 0 ? {parts[0]} : (i & 3) == 1 ? {parts[1]} : "
               f"(i & 3) == 2 ? {parts[2]} : {parts[3]}; acc = {combine.format('acc', e)}; }}")
        if init is None:
            total = combine.format(combine.format(parts[0], parts[1]), combine.format(parts[2], parts[3]))
        else:
            total = f"({parts[0]} + {parts[1]}) + ({parts[2]} + {parts[3]})"
        return b.rnew(total)


# --------------------------------------------------------------------------
# custom inputs
# --------------------------------------------------------------------------

def custom_kind(sym) -> str:
    axes = custom_axes(sym)
    if 3 in axes:
        return "tile"
    if 2 in axes:
        return "row"
    return "scalar"


def custom_ctype(sym, input_ctype: str) -> str:
    """Element type a custom tensor is read as.  As in the reference, tensors
    without a sequence axis are fp32 (e.g. ``softmax_bias`` of shape (1,),
    examples/sigmoid_attn.py:54-56) and tensors with one are in the q/k/v dtype
    (e.g. the retention mask, core/lower/lower.py:561-615)."""
    return "float" if custom_kind(sym) == "scalar" else input_ctype


def _emit_custom_loads(body: _Body, tr: TracedParallel, input_ctype: str, leaves: dict, with_tiles: bool):
    for k, (name, sym) in enumerate(tr.custom.items()):
        kind = custom_kind(sym)
        ct = custom_ctype(sym, input_ctype)
        base = (f"static_cast<const {ct}*>(c.fa->custom[{k}]) + c.b * c.fa->cstride[{k}][0] + "
                f"c.h * c.fa->cstride[{k}][1]")
        if kind == "scalar":
            v = body.fresh("cu")
            body.stmt(f"const float {v} = static_cast<float>(*({base}));")
            leaves[id(sym)] = Row(v)
        elif kind == "row":
            v = body.fresh("cu")
            body.stmt(f"const float {v} = c.q_idx < c.seq_q ? static_cast<float>(*({base} + "
                      f"static_cast<long long>(c.q_idx) * c.fa->cstride[{k}][2])) : 0.0f;")
            leaves[id(sym)] = Row(v)
        elif with_tiles:
            v = body.fresh("ct")
            p = body.fresh("cp")
            body.stmt(f"const {ct}* {p} = {base} + static_cast<long long>(c.q_idx) * c.fa->cstride[{k}][2] + "
                      f"static_cast<long long>(c.kv0) * c.fa->cstride[{k}][3];")
            body.stmt(f"float {v}[{body.n}];")
            body.stmt(f"const bool {v}_row = c.q_idx < c.seq_q;")
            body.loop(f"{v}[i] = ({v}_row && c.kv0 + i < c.seq_kv) ? static_cast<float>({p}[static_cast<long long>(i) * "
                      f"c.fa->cstride[{k}][3]]) : 0.0f;")
            leaves[id(sym)] = Tile(v)


_COMBINE_BIN = {"Add": "({0} + {1})", "Sub": "({0} - {1})", "Mul": "({0} * {1})", "Div": "({0} / {1})",
                "Max": "fmaxf({0}, {1})", "Min": "fminf({0}, {1})"}
_COMBINE_UN = {"Neg": "(-{0})", "Abs": "fabsf({0})", "Exp": f"b200::fast_exp2({{0}} * {_f(LOG2E)})", "Exp2": "b200::fast_exp2({0})",
               "Log": f"(b200::fast_log2({{0}}) * {_f(LN2)})", "Log2": "b200::fast_log2({0})", "Tanh": "b200::fast_tanh({0})"}
_COMBINE_RED = {"ColReduceSum": ("0.0f", "{0} + {1}"), "ColReduceMax": ("(-INFINITY)", "fmaxf({0}, {1})"),
                "ColReduceAbsSum": ("0.0f", "{0} + fabsf({1})")}


def emit_combine(tr: TracedParallel) -> str:
    """Body of ``combine(i, n, fin, split_stride, final_stride)``: the weight of split ``i`` among ``n`` from the
    final row scales of all splits, fin[final * final_stride + split * split_stride] -- the user's
    ``OnlineFunc.combine`` (reference: core/lower/lower_decode.py:287-302; column reductions of
    core/codegen/tl_gen.py:22-33).  A value that varies over the splits is an expression in a split index; a column
    reduction becomes a loop over the splits in front of its first use, its result one number per row."""
    if tr.combine_out is None:
        return "return 1.0f;"
    finals = list(tr.final.keys())
    leaf = {id(sym): finals.index(name) for name, sym in tr.combine_in.items()}
    lines: list[str] = []
    reduced: dict[int, str] = {}

    def expr(sym, idx: str) -> str:
        key = id(sym)
        if key in leaf:
            return f"fin[{leaf[key]} * final_stride + {idx} * split_stride]"
        if key in reduced:
            return reduced[key]
        t = sym.code.type
        if t == "Const":
            return _f(float(sym.code.value))
        if t == "Var":
            from core.lower.trace import init_value
            return _f(init_value(sym.code.name))
        if t in _COMBINE_RED:
            init, step = _COMBINE_RED[t]
            inner = expr(sym.prev[0], "k")     # may emit loops of its own first
            name = f"c{len(reduced) + 1}"
            lines.append(f"float {name} = {init};")
            lines.append(f"for (int k = 0; k < n; ++k) {name} = {step.format(name, inner)};")
            reduced[key] = name
            return name
        if t in _COMBINE_BIN:
            return _COMBINE_BIN[t].format(expr(sym.prev[0], idx), expr(sym.prev[1], idx))
        if t in _COMBINE_UN:
            return _COMBINE_UN[t].format(expr(sym.prev[0], idx))
        raise NotImplementedError(f"op {t} in OnlineFunc.combine is not supported by the functor emitter")

    result = expr(tr.combine_out, "i")
    return "\n    ".join(lines + [f"return {result};"])


@dataclass
class FunctorSource:
    struct_name: str
    code: str            # definition of the functor struct (namespace-free, uses b200:: helpers)
    n_rowscales: int
    n_final: int
    final_names: list
    custom_names: list
    unit_o_scale: bool


def emit_functor(tr: TracedParallel, *, neg_inf_mask: bool, input_ctype: str, struct_name: str = "UserFunctor") -> FunctorSource:
    rs_names = list(tr.rowscale_in.keys())
    # ---------------- tile() ----------------
    body = _Body("N")
    leaves: dict[int, object] = {id(tr.scores_in): Tile("s")}
    for k, name in enumerate(rs_names):
        v = body.fresh("in")
        body.stmt(f"const float {v} = rs[{k}];")
        leaves[id(tr.rowscale_in[name])] = Row(v)
    body.stmt("const float idx_b = static_cast<float>(c.b); const float idx_h = static_cast<float>(c.h); "
              "const float idx_q = static_cast<float>(c.q_idx);")
    leaves[id(tr.index_leaves["b"])] = Row("idx_b")
    leaves[id(tr.index_leaves["h"])] = Row("idx_h")
    leaves[id(tr.index_leaves["q_idx"])] = Row("idx_q")
    kv_leaf = tr.index_leaves["kv_idx"]
    if kv_leaf.use_list:
        body.stmt("float kvpos[N];")
        body.loop("kvpos[i] = static_cast<float>(c.kv0 + i);")
        leaves[id(kv_leaf)] = Tile("kvpos")
    _emit_custom_loads(body, tr, input_ctype, leaves, with_tiles=True)
    low = _Lowerer(body, leaves)
    new_rs = [low.lower(tr.rowscale_out[name]) for name in rs_names]
    s_out = low.lower(tr.scores_out)
    o_scale = low.lower(tr.o_scale) if tr.o_scale is not None else Const(1.0)
    if isinstance(o_scale, Tile) or any(isinstance(v, Tile) for v in new_rs):
        raise ValueError("row scales and o_scale must be per-row values")
    if not isinstance(s_out, Tile):
        body.loop(f"s[i] = {body.rexpr(s_out)};")
    elif not (s_out.name == "s" and s_out.alpha is None and s_out.beta is None):
        body.loop(f"s[i] = {body.elem(s_out)};")
    # all reads of rs[] happened at the top, so the writes below cannot alias them
    for k, v in enumerate(new_rs):
        body.stmt(f"rs[{k}] = {body.rexpr(v)};")
    body.stmt(f"return {body.rexpr(o_scale)};")
    tile_code = "\n    ".join(body.lines)

    # ---------------- epilogue() ----------------
    ebody = _Body("N")
    eleaves: dict[int, object] = {id(tr.o_in): Tile("o")}
    for k, name in enumerate(rs_names):
        eleaves[id(tr.rowscale_in[name])] = Row(f"rs[{k}]")
    ebody.stmt("const float idx_b = static_cast<float>(c.b); const float idx_h = static_cast<float>(c.h); "
               "const float idx_q = static_cast<float>(c.q_idx);")
    eleaves[id(tr.index_leaves["b"])] = Row("idx_b")
    eleaves[id(tr.index_leaves["h"])] = Row("idx_h")
    eleaves[id(tr.index_leaves["q_idx"])] = Row("idx_q")
    _emit_custom_loads(ebody, tr, input_ctype, eleaves, with_tiles=False)
    elow = _Lowerer(ebody, eleaves)
    o_out = elow.lower(tr.o_out)
    if not isinstance(o_out, Tile):
        raise ValueError("online_fwd_epilogue must return the (transformed) accumulator")
    if not (o_out.name == "o" and o_out.alpha is None and o_out.beta is None):
        ebody.loop(f"o[i] = {ebody.elem(o_out)};")
    epi_code = "\n    ".join(ebody.lines)

    # ---------------- final_rowscale() ----------------
    fbody = _Body("1")
    fleaves: dict[int, object] = {}
    for k, name in enumerate(rs_names):
        fleaves[id(tr.rowscale_in[name])] = Row(f"rs[{k}]")
    fbody.stmt("const float idx_b = static_cast<float>(c.b); const float idx_h = static_cast<float>(c.h); "
               "const float idx_q = static_cast<float>(c.q_idx);")
    fleaves[id(tr.index_leaves["b"])] = Row("idx_b")
    fleaves[id(tr.index_leaves["h"])] = Row("idx_h")
    fleaves[id(tr.index_leaves["q_idx"])] = Row("idx_q")
    _emit_custom_loads(fbody, tr, input_ctype, fleaves, with_tiles=False)
    flow = _Lowerer(fbody, fleaves)
    final_names = list(tr.final.keys())
    cases = []
    for k, name in enumerate(final_names):
        v = flow.lower(tr.final[name])
        if isinstance(v, Tile):
            raise ValueError(f"final row scale {name!r} must be a per-row value")
        cases.append(f"if (which == {k}) return {fbody.rexpr(v)};")
    final_code = "\n    ".join(fbody.lines + cases + ["return 0.0f;"])

    init_code = "\n    ".join(f"rs[{k}] = {_f(tr.rowscale_init[name])};" for k, name in enumerate(rs_names)) or "(void)rs;"
    unit = tr.o_scale is None
    code = f"""struct {struct_name} {{
  static constexpr int kRowScales = {len(rs_names)};
  static constexpr int kFinal = {len(final_names)};
  static constexpr bool kUnitOScale = {'true' if unit else 'false'};
  static constexpr bool kNegInfMask = {'true' if neg_inf_mask else 'false'};
  __device__ static void init(float* rs, const b200::RowCtx& c) {{
    {init_code}
  }}
  template <int N>
  __device__ static float tile(float (&s)[N], float* rs, const b200::RowCtx& c) {{
    {tile_code}
  }}
  template <int N>
  __device__ static void epilogue(float (&o)[N], const float* rs, const b200::RowCtx& c) {{
    {epi_code}
  }}
  __device__ static float final_rowscale(int which, const float* rs, const b200::RowCtx& c) {{
    {final_code}
  }}
  static constexpr bool kCombinedFinal = false;
  __device__ static float combined_final(int, const float*, long long, long long) {{ return 0.0f; }}
  __device__ static float combine(int i, int n, const float* fin, long long split_stride, long long final_stride) {{
    {emit_combine(tr)}
  }}
}};
"""
    return FunctorSource(struct_name, code, len(rs_names), len(final_names), final_names,
                         list(tr.custom.keys()), unit)


def translation_unit(fs: FunctorSource, dim_qk: int, dim_v: int, bf16: bool, sparse: bool = False) -> str:
    """Source of a library exporting ``attn_b200_parallel_fwd_jit`` for one functor and one
    (dim_qk, dim_v, dtype, dense or block-sparse walk) instantiation of the forward kernel."""
    b = "true" if bf16 else "false"
    dv = dim_v if dim_v <= 128 else 256    # wider dim_v runs as 128-column slices whatever its multiple
    return f"""// generated by core/lower/functor.py -- do not edit
#include "parallel_launch.cuh"

{fs.code}
extern "C" int attn_b200_parallel_fwd_jit(const AttnB200ParallelArgs* args, void* cuda_stream, int32_t* device_status) {{
  const int rc = b200::validate_parallel_args(args);
  if (rc != ATTN_B200_OK) return rc;
  if (args->dtype != {1 if bf16 else 0}) return ATTN_B200_E_UNSUPPORTED;
  if (args->dim_qk != {dim_qk} || args->dim_v != {dim_v}) return ATTN_B200_E_UNSUPPORTED;
  return b200::launch_parallel_dims<{fs.struct_name}, {dim_qk}, {dv}, {b}, {'true' if sparse else 'false'}>(
      args, static_cast<cudaStream_t>(cuda_stream), device_status);
}}
"""


def source_hash(text: str) -> str:
    return hashlib.sha256(text.encode()).hexdigest()[:20]
