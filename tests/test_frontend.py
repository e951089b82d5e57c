"""Front-end behaviour on CPU: tracing objects, pattern selection, mask
classification, pattern probing and the meaning of lowered functors (checked
through the torch interpreter of the traced DAG against the oracle)."""

import math
import os

import pytest
import torch

from conftest import reference_root
from examples_b200 import programs
from attn_engine import AttentionEngine, OnlineFunc
from core import CustomIO, SymbolicArray, SymbolScalar, Var, meta_tensor
from core.lower import functor as fl
from core.lower.trace import probe_softmax_scale, run_traced_attention, trace_parallel
from core.transform.core import create_block_mask, is_causal_mask, is_less_causal_mask
from oracle import inputs, reference_math as rm


def test_symbolic_ops_build_dag():
    s = SymbolicArray("scores", Var("scores"))
    m = SymbolScalar("m", Var("-inf"))
    m_new = m.max(s.get_reduce("max"))
    p = (s - m_new).exp()
    assert isinstance(p, SymbolicArray) and p.shape_idx == ["block_M", "block_N"]
    assert m_new.shape_idx == ["block_M"] and m_new.code.type == "Max"
    assert str(p.code).startswith("Exp(Sub(")
    assert (2.0 - s).code.type == "Sub" and (1.0 / s).code.type == "Div"
    with pytest.raises(NotImplementedError):
        p.backward()


def test_customio_decorator_registers_tensor():
    io = CustomIO({"bias": (1,)})
    io("extra", (1, "heads"))
    assert set(io.input_tensors) == {"bias", "extra"}
    with pytest.raises(ValueError):
        io("bias", (1,))


def test_block_mask_helpers():
    causal = lambda b, h, q, kv: q >= kv
    bm = create_block_mask(causal, 2, 3, 512, 512, "cpu")
    assert bm.shape == (2, 3, 4, 4) and bm.dtype == torch.int8
    assert bool(is_causal_mask(bm, 128, 128)) and bool(is_less_causal_mask(bm, 128, 128))
    window = lambda b, h, q, kv: (q >= kv) & (q - kv < 100)
    bw = create_block_mask(window, 1, 1, 512, 512, "cpu")
    assert not bool(is_causal_mask(bw, 128, 128)) and bool(is_less_causal_mask(bw, 128, 128))
    per_head = lambda b, h, q, kv: q >= kv + h
    bh = create_block_mask(per_head, 1, 2, 256, 256, "cpu", 64, 64)
    assert bh.shape == (1, 2, 4, 4)


def test_pattern_selection_follows_reference_rules():
    sel = AttentionEngine._select_pattern
    assert sel(1, 4096, 128, 1, True) == "mla_decode"
    assert sel(1, 4096, 32, 8, False) == "gqa_decode"
    assert sel(1, 4096, 16, 16, False) == "mha_decode"
    assert sel(2048, 2048, 16, 16, False) == "parallel"
    assert sel(2048, 2048, 32, 8, False) == "gqa"


def test_unsupported_patterns_raise_clearly():
    meta = (meta_tensor(1, 6, 1, 128, dtype=torch.float16), meta_tensor(1, 4, 4096, 128, dtype=torch.float16),
            meta_tensor(1, 4, 4096, 128, dtype=torch.float16))
    with pytest.raises(NotImplementedError, match="multiple of KV heads"):
        AttentionEngine(meta, CustomIO({}), None, None, None)
    meta = (meta_tensor(1, 16, 1, 128, dtype=torch.float16), meta_tensor(1, 4, 4096, 128, dtype=torch.float16),
            meta_tensor(1, 4, 4096, 128, dtype=torch.float16))
    e = AttentionEngine(meta, CustomIO({}), None, None, None, use_varlen=True, extern_block_mask=True, infer_mask_block_N=32)
    assert e.pattern == "gqa_decode" and e.custom_names == [] and e.sparse_walk   # block mask / lengths select KV tiles per call
    with pytest.raises(TypeError):
        AttentionEngine(programs._meta(1, 2, 128, 64, 64, torch.float32), CustomIO({}), None, None, None)


def test_softmax_forms_are_recognised_as_builtin():
    e = programs.softmax_engine(1, 2, 256, 64, 64)
    assert e.functor_kind == "builtin_softmax" and abs(e._fparams[0] - 0.125) < 1e-6 and e.mask_kind == 1
    e2 = programs.softmax_engine(1, 2, 256, 128, 128, is_causal=False, scale=0.3)
    assert e2.functor_kind == "builtin_softmax" and abs(e2._fparams[0] - 0.3) < 1e-6 and e2.mask_kind == 0
    assert programs.softmax_engine_noprobe(1, 2, 256, 64, 64).functor_kind == "lowered"
    assert programs.sigmoid_engine(1, 2, 256, 64, 64).functor_kind == "lowered"


def _interp(engine, q, k, v, custom=(), causal=False, neg_inf=True):
    return run_traced_attention(engine.traced, q, k, v, custom, causal=causal, neg_inf_mask=neg_inf)


def test_traced_softmax_means_softmax():
    q, k, v = inputs.attention_bshd(1, 2, 200, 64, 64, 3, dtype=torch.float32)
    e = programs.softmax_engine_noprobe(1, 2, 200, 64, 64)
    o, fin = _interp(e, q, k, v, causal=True)
    assert torch.allclose(o, rm.softmax_attention(q, k, v, True), atol=1e-5)
    assert torch.allclose(fin["lse"], rm.softmax_lse(q, k, True), atol=1e-5)


def test_traced_sigmoid_relu_retention_mean_the_reference_math():
    q, k, v = inputs.attention_bshd(1, 2, 160, 64, 64, 4, dtype=torch.float32)
    bias = torch.tensor([-2.0])
    e = programs.sigmoid_engine(1, 2, 160, 64, 64, is_causal=True)
    o, _ = _interp(e, q, k, v, (bias,), causal=True)
    assert torch.allclose(o, rm.sigmoid_attention(q, k, v, bias, True), atol=1e-5)
    o, _ = _interp(programs.relu_engine(1, 2, 160, 64, 64), q, k, v)
    assert torch.allclose(o, rm.relu_attention(q, k, v), atol=1e-4)
    mask = torch.rand(1, 2, 160, 160, generator=torch.Generator().manual_seed(1)).tril()
    e = programs.retention_parallel_engine(1, 2, 160, 64, 64)
    o, fin = _interp(e, q, k, v, (mask,), causal=True, neg_inf=False)
    assert torch.allclose(o, rm.retention_parallel(q, k, v, mask), atol=1e-5)


def test_emitted_functor_source_shape():
    e = programs.sigmoid_engine(1, 2, 256, 128, 128)
    src = e.functor_source
    assert "kUnitOScale = true" in src and "fast_tanh(fmaf(s[i]" in src
    assert "attn_b200_parallel_fwd_jit" in src
    e = programs.softmax_engine_noprobe(1, 2, 256, 64, 64)
    # exp(s*scale - m) must collapse to one FMA feeding exp2
    assert "b200::fast_exp2(fmaf(s[i]" in e.functor_source and "kFinal = 2" in e.functor_source


def test_engine_needs_cuda_tensors():
    e = programs.softmax_engine(1, 2, 128, 64, 64)
    q, k, v = inputs.attention_bshd(1, 2, 128, 64, 64, 1)
    with pytest.raises(Exception):
        e(q, k, v)   # CPU tensors: there is no CPU fallback


@pytest.mark.skipif(reference_root() is None, reason="reference checkout not present")
def test_reference_examples_construct_unchanged():
    """The reference's own example programs run unchanged on top of this package."""
    import importlib
    import sys
    ref = reference_root()
    sys.path.insert(0, ref)
    try:
        mha = importlib.import_module("examples.mha")
        assert mha.causal_softmax_attention(1, 4, 512, 128, 128, dtype=torch.bfloat16).functor_kind == "builtin_softmax"
        v2 = importlib.import_module("examples.mha_v2")
        assert v2.causal_softmax_attention(1, 4, 512, 128, 128).functor_kind == "builtin_softmax"
        sg = importlib.import_module("examples.sigmoid_attn")
        assert sg.sigmoid_attention(1, 4, 512, 128, 128).functor_kind == "lowered"
        sg2 = importlib.import_module("examples.sigmoid_attn_v2")
        assert sg2.sigmoid_attention(1, 4, 512, 128, 128).functor_kind == "lowered"
        relu = importlib.import_module("examples.reluattn")
        assert relu.relu_attention(1, 6, 512, 64, 64).mask_kind == 0
        ret = importlib.import_module("examples.retnet_recurrent")
        assert ret.retnet_recurrent(1, 8, 512, 256, 512).q_scale == 256 ** -0.5
        gla = importlib.import_module("examples.gated_retention")
        assert gla.gated_retention(1, 4, 512, 256, 256).q_scale == 1 / 256 ** 0.5
        rp = importlib.import_module("examples.retention_parallel")
        assert rp.retention_parallel(1, 32, 2048, 256, 512).functor_kind == "lowered"   # the README's smoke run
        sp = importlib.import_module("examples.sparse_gqa_decode")
        assert sp.sparse_gqa_decode(2, 32, 8, 4096, 128, 128).pattern == "gqa_decode"
        dec = importlib.import_module("examples.mha_decode")
        assert dec.softmax_attention_decode(2, 8, 1, 4096, 128, 128).pattern == "mha_decode"
        mb = importlib.import_module("examples.mamba2")
        e = mb.mamba2(1, 1, 512, 128, 64, HK=1, HV=8)
        assert e.custom_names == ["A", "dt"] and e.H == 8 and e.HK == 1
    finally:
        sys.path.remove(ref)


def test_band_masks_are_recognised():
    from attn_engine.attn_engine import classify_mask
    from core.native import lib as native
    assert classify_mask(programs.sliding_window_mask, 1, 2, 512, 512) == (native.MASK_BAND, (127, 0))
    assert classify_mask(lambda b, h, q, kv: (kv - q <= 40) & (q - kv <= 70), 1, 1, 300, 300) == (native.MASK_BAND, (70, 40))
    assert classify_mask(lambda b, h, q, kv: kv <= q + 5, 1, 1, 200, 200) == (native.MASK_BAND, (native.MASK_OPEN, 5))
    assert classify_mask(programs.causal, 1, 1, 256, 256)[0] == native.MASK_CAUSAL
    assert classify_mask(lambda b, h, q, kv: q >= 0, 1, 1, 128, 128)[0] == native.MASK_NONE
    from attn_engine.attn_engine import MASK_GENERAL
    assert classify_mask(lambda b, h, q, kv: (q + kv) % 2 == 0, 1, 1, 128, 128)[0] == MASK_GENERAL   # not a band
    assert classify_mask(lambda b, h, q, kv: (kv <= q) & (h >= 0) & (b == 0), 2, 1, 128, 128)[0] == MASK_GENERAL   # uses the batch index


def test_general_masks_become_block_sparse_walks():
    """Bitmaps and element masks of a mask that is not a band, against the dense mask they stand for."""
    from core.lower import sparse
    import numpy as np
    doc = lambda b, h, q, kv: (q // 192 == kv // 192) & (q >= kv)      # causal inside documents of 192 tokens
    S = 600
    sp = sparse.build_block_sparse(doc, 2, 3, S, S)
    assert (sp["batch"], sp["heads"], sp["mask_rows"]) == (1, 1, 128) and sp["keep"].shape == (1, 1, 5, 1)
    dense = doc(0, 0, torch.arange(S).view(-1, 1), torch.arange(S).view(1, -1))
    rebuilt = torch.zeros(640, 640, dtype=torch.bool)
    keep = sp["keep"].numpy().view(np.uint32)
    part = sp["partial"].numpy().view(np.uint32)
    elem = sp["elem_mask"].numpy().view(np.uint32)
    for qt in range(5):
        slot = int(sp["mask_base"][0, 0, qt])
        for kt in range(5):
            if not (keep[0, 0, qt, 0] >> kt) & 1:
                continue
            if (part[0, 0, qt, 0] >> kt) & 1:
                bits = (elem[slot][:, :, None] >> np.arange(32, dtype=np.uint32)) & 1      # [128, 4, 32]
                rebuilt[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128] = torch.from_numpy(bits.reshape(128, 128).astype(bool))
                slot += 1
            else:
                rebuilt[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128] = True
    assert torch.equal(rebuilt[:S, :S], dense)
    assert sp["kept_tiles"] < sp["all_tiles"]
    # the kept tiles are those of the reference's block mask
    assert torch.equal(torch.from_numpy(((keep[0, 0, :, 0, None] >> np.arange(5, dtype=np.uint32)) & 1).astype(np.int8)),
                       create_block_mask(doc, 1, 1, S, S, "cpu")[0, 0])
    per_head = sparse.build_block_sparse(lambda b, h, q, kv: q >= kv + 64 * h, 2, 3, 256, 256)
    assert (per_head["batch"], per_head["heads"]) == (2, 3)
    e = programs.masked_softmax_engine(1, 2, 384, 64, 64, doc)
    assert e.sparse_walk and e.functor_kind == "builtin_softmax" and e.mask_kind == 0


def _softmax_with_score_mod(score_mod, S=256, D=64):
    return AttentionEngine(programs._meta(1, 2, S, D, D, torch.bfloat16), CustomIO({}), score_mod=score_mod,
                           mask_mod=programs.causal, online_func=programs.NaturalSoftmax())


def test_look_alikes_of_softmax_are_lowered_not_recognised():
    """Only DAGs that can be nothing but online softmax reach the built-in functor: a soft cap (tanh saturates only for
    large logits), a relative bias that starts far from the diagonal, a per-head slope or a custom bias all look like
    softmax on a small random probe and must be lowered."""
    for cap in (50.0, 100.0):
        e = _softmax_with_score_mod(lambda s, c, b, h, q, kv, cap=cap: (s * 0.125 / cap).tanh() * cap)
        assert e.functor_kind == "lowered"
    far = _softmax_with_score_mod(lambda s, c, b, h, q, kv: s * 0.125 - ((q - kv) - 64.0).max(0.0) * 0.5)
    assert far.functor_kind == "lowered"
    slope = _softmax_with_score_mod(lambda s, c, b, h, q, kv: s * 0.125 + h * 0.0)
    assert slope.functor_kind == "lowered"
    plain = _softmax_with_score_mod(lambda s, c, b, h, q, kv: s / 8.0)
    assert plain.functor_kind == "builtin_softmax" and abs(plain._fparams[0] - 0.125) < 1e-6


def test_mask_dependence_on_batch_or_head_is_decided_by_use():
    from core.transform.core import mask_depends_on_batch_head
    assert not mask_depends_on_batch_head(programs.causal, 4, 9, 512, 512)
    assert not mask_depends_on_batch_head(programs.sliding_window_mask, 4, 9, 512, 512)
    # differs only at one head in the middle of the range: corner sampling would miss it
    assert mask_depends_on_batch_head(lambda b, h, q, kv: (q >= kv) | (h == 4), 4, 9, 512, 512)
    assert mask_depends_on_batch_head(lambda b, h, q, kv: (q >= kv) & (b >= 0), 4, 9, 512, 512)


def test_custom_input_shapes_are_checked_before_launch():
    e = programs.retention_parallel_engine(1, 2, 256, 64, 64)          # mask declared (1, heads, seq_len, seq_len_kv)
    ok = torch.zeros(1, 2, 256, 256)
    tensors, strides = e._custom_operands((ok,), 1, 2, 256, 256, torch.device("cpu"))
    assert strides[0] == [0, 256 * 256, 256, 1]
    e._custom_operands((torch.zeros(1, 1, 256, 256),), 1, 2, 256, 256, torch.device("cpu"))   # broadcast over heads
    for bad in (torch.zeros(1, 2, 256, 255), torch.zeros(1, 2, 200, 256), torch.zeros(2, 256, 256), torch.zeros(2, 2, 256, 256)):
        with pytest.raises(ValueError):
            e._custom_operands((bad,), 1, 2, 256, 256, torch.device("cpu"))
    s = programs.sigmoid_engine(1, 2, 256, 64, 64)
    with pytest.raises(ValueError):
        s._custom_operands((torch.zeros(3),), 1, 2, 256, 256, torch.device("cpu"))


def test_operands_on_different_devices_are_refused():
    e = programs.softmax_engine(1, 2, 128, 64, 64)
    q, k, v = inputs.attention_bshd(1, 2, 128, 64, 64, 1)
    with pytest.raises(ValueError, match="one device"):
        e._run_parallel_impl(q, k.to("meta"), v)
