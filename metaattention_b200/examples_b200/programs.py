"""User-level programs against the AttentionEngine API, written for the tests
and the benchmark (the reference's examples/*.py are exercised directly from
the reference checkout where one is present; these cover the same patterns)."""

import math

import torch
from attn_engine import AttentionEngine, LinearAttentionEngine, OnlineFunc
from core import CustomIO, SymbolScalar, Var, meta_tensor


def _meta(B, H, S, D, Dv, dtype):
    return (meta_tensor(B, H, S, D, dtype=dtype), meta_tensor(B, H, S, D, dtype=dtype),
            meta_tensor(B, H, S, Dv, dtype=dtype))


def causal(b, h, q_idx, kv_idx):
    return q_idx >= kv_idx


class NaturalSoftmax(OnlineFunc):
    """Online softmax with natural exponentials on pre-scaled scores."""

    def __init__(self):
        super().__init__({"m": SymbolScalar("m", Var("-inf")), "r": SymbolScalar("r", Var("0.0"))},
                         {"lse": SymbolScalar("lse", Var("0.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        m, r = online_rowscales["m"], online_rowscales["r"]
        m_new = m.max(scores.get_reduce("max"))
        shrink = (m - m_new).exp()
        p = (scores - m_new).exp()
        return p, {"m": m_new, "r": r * shrink + p.get_reduce("sum")}, shrink

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        r, m = online_rowscales["r"], online_rowscales["m"]
        return o / r, {"lse": r.log() + m}


def softmax_engine(B, H, S, D, Dv, dtype=torch.bfloat16, is_causal=True, scale=None):
    scale = D ** -0.5 if scale is None else scale

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({}), score_mod=score_mod,
                           mask_mod=causal if is_causal else None, online_func=NaturalSoftmax())


def softmax_engine_noprobe(B, H, S, D, Dv, dtype=torch.bfloat16, is_causal=True):
    """Same math, but with a second (unused by the output) final row scale so that the
    built-in softmax functor is NOT selected: exercises the generic lowering of an online
    function with running row scales and accumulator rescaling."""
    scale = D ** -0.5

    class TwoFinals(NaturalSoftmax):
        def __init__(self):
            OnlineFunc.__init__(self, {"m": SymbolScalar("m", Var("-inf")), "r": SymbolScalar("r", Var("0.0"))},
                                {"lse": SymbolScalar("lse", Var("0.0")), "rowmax": SymbolScalar("rowmax", Var("0.0"))},
                                CustomIO())

        @staticmethod
        def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
            r, m = online_rowscales["r"], online_rowscales["m"]
            return o / r, {"lse": r.log() + m, "rowmax": m}

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({}), score_mod=score_mod,
                           mask_mod=causal if is_causal else None, online_func=TwoFinals())


def sigmoid_engine(B, H, S, D, Dv, dtype=torch.bfloat16, is_causal=False, scale=1.0, online="identity"):
    """score = sigmoid(scale * q.k + bias) in tanh form; ``bias`` is a (1,) fp32 custom input."""

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        x = score * scale + custom.input_tensors["softmax_bias"]
        return ((x * 0.5).tanh() + 1) * 0.5
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({"softmax_bias": (1,)}), score_mod=score_mod,
                           mask_mod=causal if is_causal else None,
                           online_func=None if online is None else OnlineFunc({}, {}, CustomIO()))


def relu_engine(B, H, S, D, Dv, dtype=torch.bfloat16):
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return (score * scale).max(0)
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({}), score_mod=score_mod, mask_mod=None,
                           online_func=None)


class AbsSumNormaliser(OnlineFunc):
    """Retention's normaliser: divide by max(running sum of |scores|, 1)."""

    def __init__(self):
        super().__init__({"acc": SymbolScalar("acc", Var("0.0")), "den": SymbolScalar("den", Var("0.0"))},
                         {"den": SymbolScalar("den", Var("0.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        acc = online_rowscales["acc"] + scores.get_reduce("abssum")
        den_new = acc.max(1.0)
        return scores / den_new, {"acc": acc, "den": den_new}, online_rowscales["den"] / den_new

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, {"den": online_rowscales["den"]}


def retention_parallel_engine(B, H, S, D, Dv, dtype=torch.bfloat16):
    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * custom.input_tensors["mask"]
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({"mask": (1, "heads", "seq_len", "seq_len_kv")}),
                           score_mod=score_mod, mask_mod=causal, online_func=AbsSumNormaliser(), mask_value="0")


def mla_engine(B, H, S, D, Dv, dtype=torch.bfloat16, backend="tl"):
    """MLA decode engine: one query token, a single latent KV head shared by all query heads."""
    meta = (meta_tensor(B, H, 1, D, dtype=dtype), meta_tensor(B, 1, S, D, dtype=dtype), meta_tensor(B, 1, S, Dv, dtype=dtype))
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    return AttentionEngine(meta, CustomIO({}), score_mod=score_mod, mask_mod=None, online_func=NaturalSoftmax(),
                           kv_shared=True, backend=backend)


def retnet_engine(B, H, S, Dk, Dv, dtype=torch.bfloat16):
    """RetNet retention in the chunked pattern: decay holds gamma_h, decay_mod takes its log,
    q is scaled by 1/sqrt(Dk)."""
    scale = Dk ** -0.5

    def decay_mod(decay, custom_io):
        return decay.log()

    def q_mod(q, custom_io):
        return q * scale
    meta = (meta_tensor(B, H, S, Dk, dtype=dtype), meta_tensor(B, H, S, Dk, dtype=dtype), meta_tensor(B, H, S, Dv, dtype=dtype))
    return LinearAttentionEngine(meta, q_mod=q_mod, decay_mod=decay_mod, custom_io=CustomIO({}))


def gla_engine(B, H, S, D, Dv, dtype=torch.bfloat16):
    """Gated retention / simple GLA as examples/gated_retention.py builds it: q scaled by 1/sqrt(D),
    the decay input already holds the per-token natural-log decay."""
    scale = 1 / D ** 0.5

    def q_mod(q, custom_io):
        return q * scale
    meta = (meta_tensor(B, H, S, D, dtype=dtype), meta_tensor(B, H, S, D, dtype=dtype), meta_tensor(B, H, S, Dv, dtype=dtype))
    return LinearAttentionEngine(meta, q_mod=q_mod, custom_io=CustomIO({}))


def mamba2_engine(B, HQ, S, D, Dv, HK=None, HV=None, dtype=torch.bfloat16):
    """Mamba2 SSD as examples/mamba2.py builds it: decay_mod = decay * A, v_mod = v * dt;
    called as mod(q, k, v, dt, A, dt)."""
    HK = HQ if HK is None else HK
    HV = HQ if HV is None else HV

    def decay_mod(decay, custom_io):
        A = custom_io.input_tensors["A"]
        return (decay * A)

    def v_mod(v, custom_io):
        dt = custom_io.input_tensors["dt"]
        return v * dt
    meta = (meta_tensor(B, HQ, S, D, dtype=dtype), meta_tensor(B, HK, S, D, dtype=dtype), meta_tensor(B, HV, S, Dv, dtype=dtype))
    custom_io = CustomIO({"A": (1, "heads"), "dt": ("batch", "heads", "seq_len")})
    return LinearAttentionEngine(meta, decay_mod=decay_mod, v_mod=v_mod, custom_io=custom_io)


def softmax_decode_engine(B, H, Sq, Skv, D, Dv, dtype=torch.bfloat16):
    """A few query rows against a long KV, built like examples/mha_decode.py: the q meta tensor is padded to
    a multiple of 128 rows, no mask."""
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    meta = (meta_tensor(B, H, ((Sq + 127) // 128) * 128, D, dtype=dtype), meta_tensor(B, H, Skv, D, dtype=dtype),
            meta_tensor(B, H, Skv, Dv, dtype=dtype))
    return AttentionEngine(meta, CustomIO({}), score_mod=score_mod, mask_mod=None, online_func=NaturalSoftmax())


def gqa_engine(B, H, Hkv, Sq, Skv, D, Dv, dtype=torch.bfloat16, is_causal=False):
    """Grouped KV heads: H query heads share Hkv KV heads (prefill when Sq == Skv, dense decode otherwise)."""
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    meta = (meta_tensor(B, H, Sq, D, dtype=dtype), meta_tensor(B, Hkv, Skv, D, dtype=dtype), meta_tensor(B, Hkv, Skv, Dv, dtype=dtype))
    return AttentionEngine(meta, CustomIO({}), score_mod=score_mod, mask_mod=causal if is_causal else None,
                           online_func=NaturalSoftmax())


def sliding_window_mask(b, h, q_idx, kv_idx):
    """the mask of the reference's tracing test (attention_engine/tests/test_torchtrace.py:5-6)"""
    return torch.logical_and(q_idx >= kv_idx, q_idx < kv_idx + 128)


def masked_softmax_engine(B, H, S, D, Dv, mask_mod, dtype=torch.bfloat16):
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({}), score_mod=score_mod, mask_mod=mask_mod,
                           online_func=NaturalSoftmax())


def sparse_decode_engine(B, H, Hkv, Skv, D, Dv, block=32, dtype=torch.bfloat16):
    """Block-sparse, variable-length GQA decode built like examples/sparse_gqa_decode.py: no mask_mod, the kept
    blocks and the sequence lengths arrive with each call (block_mask=, cache_seqlens=)."""
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    meta = (meta_tensor(B, H, 1, D, dtype=dtype), meta_tensor(B, Hkv, Skv, D, dtype=dtype), meta_tensor(B, Hkv, Skv, Dv, dtype=dtype))
    return AttentionEngine(meta, CustomIO({}), score_mod=score_mod, mask_mod=None, online_func=NaturalSoftmax(),
                           extern_block_mask=True, use_varlen=True, infer_mask_block_N=block)


class Base2Softmax(OnlineFunc):
    """Online softmax written with base-2 exponentials and logarithms on scores that are already scaled."""
    LOG2E, LN2 = 1.4426950408889634, 0.6931471805599453

    def __init__(self):
        super().__init__({"m": SymbolScalar("m", Var("-inf")), "r": SymbolScalar("r", Var("0.0"))},
                         {"lse": SymbolScalar("lse", Var("0.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        m, r = online_rowscales["m"], online_rowscales["r"]
        m_new = m.max(scores.get_reduce("max"))
        shrink = ((m - m_new) * Base2Softmax.LOG2E).exp2()
        p = ((scores - m_new) * Base2Softmax.LOG2E).exp2()
        return p, {"m": m_new, "r": r * shrink + p.get_reduce("sum")}, shrink

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        r, m = online_rowscales["r"], online_rowscales["m"]
        return o / r, {"lse": r.log2() * Base2Softmax.LN2 + m}


def capped_distance_bias_engine(B, H, S, D, Dv, cap=2.0, slope=0.02, dtype=torch.bfloat16):
    """Causal softmax of min(scale * q.k, cap) - slope_h * |q_idx - kv_idx| with slope_h = slope * (h + 1): a logit
    cap and a per-head linear distance bias.  Drives Min, Abs, Neg, index operands, Exp2, Log2 and a division by a
    per-row value through the lowered functor."""
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        dist = (q_idx - kv_idx).abs()
        return (score * scale).min(cap) + (-dist) * ((h + 1) * slope)
    return AttentionEngine(_meta(B, H, S, D, Dv, dtype), CustomIO({}), score_mod=score_mod, mask_mod=causal,
                           online_func=Base2Softmax())


class SplitSoftmax(NaturalSoftmax):
    """Online softmax with the split-KV ``combine`` of examples/mha_decode.py, written with natural exponentials so
    that it matches the natural-log lse of the epilogue: w_i = exp(lse_i - log sum_k exp(lse_k)).  A second final row
    scale keeps the engine from recognising the built-in softmax, so the combine below is what runs."""

    def __init__(self):
        OnlineFunc.__init__(self, {"m": SymbolScalar("m", Var("-inf")), "r": SymbolScalar("r", Var("0.0"))},
                            {"lse": SymbolScalar("lse", Var("0.0")), "rowmax": SymbolScalar("rowmax", Var("0.0"))},
                            CustomIO())

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        r, m = online_rowscales["r"], online_rowscales["m"]
        return o / r, {"lse": r.log() + m, "rowmax": m}

    @staticmethod
    def combine(final_rowscales):
        lse = final_rowscales["lse"]
        lse_max = lse.get_reduce("max")
        total = (lse - lse_max).exp().get_reduce("sum")
        return (lse - (total.log() + lse_max)).exp()


class SplitAbsSum(OnlineFunc):
    """A normaliser that is not softmax: p = scores / max(running sum of |scores|, 1) like retention's, with a
    ``combine`` that re-normalises the splits by their denominators: w_i = den_i / max(sum_k acc_k, 1)."""

    def __init__(self):
        super().__init__({"acc": SymbolScalar("acc", Var("0.0")), "den": SymbolScalar("den", Var("1.0"))},
                         {"acc": SymbolScalar("acc", Var("0.0")), "den": SymbolScalar("den", Var("1.0"))}, CustomIO())

    @staticmethod
    def online_fwd(scores, online_rowscales, b, h, q_idx):
        acc = online_rowscales["acc"] + scores.get_reduce("abssum")
        den_new = acc.max(1.0)
        return scores / den_new, {"acc": acc, "den": den_new}, online_rowscales["den"] / den_new

    @staticmethod
    def online_fwd_epilogue(o, online_rowscales, b, h, q_idx):
        return o, {"acc": online_rowscales["acc"], "den": online_rowscales["den"]}

    @staticmethod
    def combine(final_rowscales):
        acc, den = final_rowscales["acc"], final_rowscales["den"]
        return den / acc.get_reduce("abssum").max(1.0)


def split_decode_engine(B, H, Sq, Skv, D, Dv, online="softmax", dtype=torch.bfloat16):
    """Decode (a few query rows against a long KV, no mask) through a LOWERED functor with its own combine."""
    scale = D ** -0.5

    def score_mod(score, custom, b, h, q_idx, kv_idx):
        return score * scale
    meta = (meta_tensor(B, H, ((Sq + 127) // 128) * 128, D, dtype=dtype), meta_tensor(B, H, Skv, D, dtype=dtype),
            meta_tensor(B, H, Skv, Dv, dtype=dtype))
    return AttentionEngine(meta, CustomIO({}), score_mod=score_mod, mask_mod=None,
                           online_func=SplitSoftmax() if online == "softmax" else SplitAbsSum())
