"""Backward of softmax attention (attn_b200_softmax_bwd and the engine's autograd path) against the committed
gradients of the reference's own closure (tests/golden/softmax_bwd_*.pt: torch autograd through testing/test.py:79-104,
the comparison the reference's test makes at :106-127) and against the CPU oracle on further shapes.
Tolerances for 16-bit results against fp32: max-abs 2e-2, mean-abs 2e-3."""

import os

import pytest
import torch

from oracle import inputs, reference_math as rm

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def check(got, want, what):
    """max-abs 2e-2 and mean-abs 2e-3, scaled by the magnitude of the expected tensor where that exceeds 1: the
    maximum by its largest value, the mean by 1.5 x its standard deviation (rounding a result of standard deviation s to
    bf16 costs a mean-abs error of 2.2e-3 s by itself; gradients summed over a group of heads, over hundreds of
    un-normalised sigmoid weights, or with the larger scale of head dim 64 have s = 2-4)."""
    d = (got.float().cpu() - want.float()).abs()
    assert torch.isfinite(got).all(), what
    assert d.max().item() <= MAX_ABS * max(1.0, want.abs().max().item()), (what, d.max().item(), want.abs().max().item())
    assert d.mean().item() <= MEAN_ABS * max(1.0, 1.5 * want.std().item()), (what, d.mean().item(), want.std().item())


def native_forward(q, k, v, causal, scale):
    from core.native import lib
    B, S, H, _ = q.shape
    o = torch.empty((B, S, H, v.shape[-1]), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    args = lib.fill_parallel_args(q, k, v, o, mask_kind=lib.MASK_CAUSAL if causal else lib.MASK_NONE,
                                  functor=lib.FUNCTOR_SOFTMAX, fparams=(scale,), final_rowscales=[lse])
    lib.parallel_fwd(args)
    return o, lse


@pytest.mark.parametrize("name", ["softmax_bwd_causal", "softmax_bwd_noncausal"])
def test_against_reference_golden(name):
    from core.native import lib
    g = torch.load(os.path.join(GOLD, f"{name}.pt"))
    B, H, S, D, Dv = g["shape"]
    q, k, v = (t.cuda() for t in inputs.attention_bshd(B, H, S, D, Dv, g["seed"]))
    scale = D ** -0.5
    o, lse = native_forward(q, k, v, g["causal"], scale)
    dq, dk, dv = lib.softmax_bwd(q, k, v, o, lse, g["d_o"].cuda(), scale, lib.MASK_CAUSAL if g["causal"] else lib.MASK_NONE)
    torch.cuda.synchronize()
    assert lib.last_device_status() == 0
    check(o, g["o"], "o")
    check(dq, g["dq"], "dq")
    check(dk, g["dk"], "dk")
    check(dv, g["dv"], "dv")


@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,causal,dtype", [
    (1, 2, 2, 128, 128, False, torch.float16),     # one tile
    (2, 4, 4, 512, 512, True, torch.bfloat16),     # several tiles, the diagonal ones masked
    (1, 2, 2, 300, 300, True, torch.bfloat16),     # ragged last tile
    (1, 4, 2, 384, 384, True, torch.bfloat16),     # grouped KV heads: dk, dv sum over the group
    (1, 2, 1, 200, 333, False, torch.bfloat16),    # different lengths, both ragged
    (1, 2, 2, 100, 700, False, torch.float16),     # one query tile against many KV tiles
    (1, 1, 1, 640, 256, True, torch.bfloat16),     # causal with more queries than keys (kv <= q: top-left aligned)
])
@pytest.mark.parametrize("D", [128, 64])
def test_shapes_against_oracle(B, H, Hkv, Sq, Skv, causal, dtype, D):
    from core.native import lib
    g = torch.Generator().manual_seed(Sq * 7 + Skv)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype)
    v = torch.randn(B, Skv, Hkv, D, generator=g).to(dtype)
    d_o = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    scale = D ** -0.5
    keep = None
    if causal and Sq != Skv:
        keep = torch.arange(Skv)[None, :] <= torch.arange(Sq)[:, None]
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        rm.softmax_attention(qf, kf, vf, causal, scale, keep=keep).backward(d_o.float())
    o, lse = native_forward(q.cuda(), k.cuda(), v.cuda(), causal, scale)
    dq, dk, dv = lib.softmax_bwd(q.cuda(), k.cuda(), v.cuda(), o, lse, d_o.cuda(), scale,
                                 lib.MASK_CAUSAL if causal else lib.MASK_NONE)
    torch.cuda.synchronize()
    assert lib.last_device_status() == 0
    check(dq, qf.grad, "dq")
    check(dk, kf.grad, "dk")
    check(dv, vf.grad, "dv")


def test_results_are_reproducible():
    """No atomics anywhere: two runs give the same bits."""
    from core.native import lib
    q, k, v = (t.cuda() for t in inputs.attention_bshd(2, 3, 384, 128, 128, 7))
    d_o = torch.randn(2, 384, 3, 128, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).cuda()
    o, lse = native_forward(q, k, v, True, 128 ** -0.5)
    a = lib.softmax_bwd(q, k, v, o, lse, d_o, 128 ** -0.5, lib.MASK_CAUSAL)
    b = lib.softmax_bwd(q, k, v, o, lse, d_o, 128 ** -0.5, lib.MASK_CAUSAL)
    torch.cuda.synchronize()
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("causal", [False, True])
def test_engine_autograd(causal):
    """The user's path: the traced softmax program (score_mod = scale, the softmax online_func) with tensors that
    require gradients, `o.backward(d_o)` as in the reference's examples/mha.py."""
    from examples_b200 import programs
    B, H, S, D = 1, 4, 320, 128
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 33)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(34)).to(torch.bfloat16)
    want = rm.softmax_attention_grads(q, k, v, d_o, causal, D ** -0.5)
    eng = programs.softmax_engine(B, H, S, D, D, is_causal=causal)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), rm.softmax_attention(q, k, v, causal, D ** -0.5), "o")
    for got, ref, what in zip((qc.grad, kc.grad, vc.grad), want, ("dq", "dk", "dv")):
        check(got, ref, what)


def test_programs_without_a_backward_say_so():
    from examples_b200 import programs
    B, H, S, D, Dv = 1, 2, 128, 192, 128
    q, k, v = (t.cuda().requires_grad_() for t in inputs.attention_bshd(B, H, S, D, Dv, 35))
    eng = programs.softmax_engine(B, H, S, D, Dv, is_causal=True)   # head dims 192 / 128: forward only
    o = eng(q, k, v)
    with pytest.raises(NotImplementedError):
        o.sum().backward()


@pytest.mark.parametrize("program,D,Dv,dtype", [("softmax", 128, 256, torch.float16), ("softmax", 128, 384, torch.bfloat16),
                                                ("relu", 128, 256, torch.bfloat16)])
def test_dim_v_a_multiple_of_dim_qk(program, D, Dv, dtype):
    """The reference's suite differentiates causal softmax with head dims 128 / 256 in fp16 (testing/test.py:55,
    73-127): one backward per dim_qk-wide column slice of v, dQ and dK added up."""
    from examples_b200 import programs
    B, H, S = 1, 3, 400
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, 41, dtype=dtype, k_scale=0.5 if program == "relu" else 1.0,
                                    v_scale=0.5 if program == "relu" else 1.0)
    d_o = torch.randn(B, S, H, Dv, generator=torch.Generator().manual_seed(42)).to(dtype)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        ref = rm.softmax_attention(qf, kf, vf, True, D ** -0.5) if program == "softmax" else rm.relu_attention(qf, kf, vf)
        ref.backward(d_o.float())
    eng = (programs.softmax_engine(B, H, S, D, Dv, dtype=dtype, is_causal=True) if program == "softmax"
           else programs.relu_engine(B, H, S, D, Dv, dtype=dtype))
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), ref.detach(), "o")
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        assert got.shape == want.shape, what
        check(got, want, what)


def test_argument_errors():
    from core.native import lib
    a = lib.SoftmaxBwdArgs()
    assert lib.load_library().attn_b200_softmax_bwd_workspace_bytes(None) == -1
    assert lib.load_library().attn_b200_softmax_bwd(None, None) != 0
    assert lib.load_library().attn_b200_softmax_bwd(a, None) != 0   # null tensors


# ---------------------------------------------------------------------------------------------------------------
# elementwise programs: the backward functor is derived from the traced score_mod and compiled on first use
# ---------------------------------------------------------------------------------------------------------------

def test_sigmoid_attention_against_reference_golden():
    """examples/sigmoid_attn.py differentiated: gradients of the reference's own closure (testing/test.py:519-543) by
    torch autograd, committed as tests/golden/sigmoid_bwd.pt."""
    from examples_b200 import programs
    g = torch.load(os.path.join(GOLD, "sigmoid_bwd.pt"))
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"])
    eng = programs.sigmoid_engine(B, H, S, D, Dv, is_causal=g["causal"], scale=D ** -0.5)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc, torch.tensor([g["bias"]]).cuda())
    o.backward(g["d_o"].cuda())
    torch.cuda.synchronize()
    check(o.detach(), g["o"], "o")
    check(qc.grad, g["dq"], "dq")
    check(kc.grad, g["dk"], "dk")
    check(vc.grad, g["dv"], "dv")


@pytest.mark.parametrize("causal,S,H,Hkv", [(False, 300, 2, 2), (True, 384, 4, 4)])
def test_sigmoid_attention_shapes(causal, S, H, Hkv):
    from examples_b200 import programs
    B, D = 1, 128
    g = torch.Generator().manual_seed(S)
    q = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, generator=g).to(torch.bfloat16)
    d_o = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    bias = torch.tensor([-2.0])
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        g_ = H // Hkv   # query head h reads KV head h // g_: the shared heads' gradients add up
        rm.sigmoid_attention(qf * D ** -0.5, kf.repeat_interleave(g_, 2), vf.repeat_interleave(g_, 2), bias, causal).backward(d_o.float())
    eng = programs.sigmoid_engine(B, H, S, D, D, is_causal=causal, scale=D ** -0.5)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    eng(qc, kc, vc, bias.cuda()).backward(d_o.cuda())
    torch.cuda.synchronize()
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        check(got, want, what)


def test_relu_attention():
    """examples/reluattn.py (relu of the scaled scores, head dim 64): the derivative is a comparison."""
    from examples_b200 import programs
    B, H, S, D = 1, 3, 192, 64
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 31, k_scale=0.5, v_scale=0.5)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(32)).to(torch.bfloat16)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        rm.relu_attention(qf, kf, vf).backward(d_o.float())
    eng = programs.relu_engine(B, H, S, D, D)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    eng(qc, kc, vc).backward(d_o.cuda())
    torch.cuda.synchronize()
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        check(got, want, what)


@pytest.mark.parametrize("left,right,Sq,Skv", [(127, 0, 700, 700),      # the sliding window of the reference's tracing test
                                               (200, 0, 512, 512),      # window edges inside tiles
                                               (64, 32, 400, 400),      # a band around the diagonal
                                               (300, 300, 384, 640)])   # wide band, more keys than queries
def test_band_masks_against_oracle(left, right, Sq, Skv):
    """Sliding windows (ATTN_B200_MASK_BAND, keep q - left <= kv <= q + right): tile pairs outside the band are skipped
    in both launches, pairs an edge crosses are masked element by element; against autograd over the oracle with the
    same keep matrix (the reference's backward applies any mask_mod element-wise, attn_tl.py:430-461)."""
    from core.native import lib
    B, H, D, dtype = 1, 2, 128, torch.bfloat16
    g = torch.Generator().manual_seed(left * 7 + right)
    q = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    k = torch.randn(B, Skv, H, D, generator=g).to(dtype)
    v = torch.randn(B, Skv, H, D, generator=g).to(dtype)
    d_o = torch.randn(B, Sq, H, D, generator=g).to(dtype)
    scale = D ** -0.5
    qi, ki = torch.arange(Sq)[:, None], torch.arange(Skv)[None, :]
    keep = (ki >= qi - left) & (ki <= qi + right)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        rm.softmax_attention(qf, kf, vf, False, scale, keep=keep).backward(d_o.float())
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty_like(qc)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device="cuda")
    args = lib.fill_parallel_args(qc, kc, vc, o, mask_kind=lib.MASK_BAND, mask_band=(left, right), functor=lib.FUNCTOR_SOFTMAX,
                                  fparams=(scale,), final_rowscales=[lse])
    lib.parallel_fwd(args)
    dq, dk, dv = lib.softmax_bwd(qc, kc, vc, o, lse, d_o.cuda(), scale, lib.MASK_BAND, (left, right))
    torch.cuda.synchronize()
    assert lib.last_device_status() == 0
    check(dq, qf.grad, "dq")
    check(dk, kf.grad, "dk")
    check(dv, vf.grad, "dv")


def test_sliding_window_engine_autograd():
    """A traced mask_mod that is a sliding window (attention_engine/tests/test_torchtrace.py:5-6) with softmax: the
    engine classifies it as a band and differentiates it."""
    from examples_b200 import programs
    B, H, S, D = 1, 2, 520, 128
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 51)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(52)).to(torch.bfloat16)
    qi, ki = torch.arange(S)[:, None], torch.arange(S)[None, :]
    keep = (qi >= ki) & (qi < ki + 128)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        ref = rm.softmax_attention(qf, kf, vf, False, D ** -0.5, keep=keep)
        ref.backward(d_o.float())
    eng = programs.masked_softmax_engine(B, H, S, D, D, programs.sliding_window_mask)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), ref.detach(), "o")
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        check(got, want, what)


@pytest.mark.parametrize("which", ["document", "checker"])
def test_general_masks_through_the_engine(which):
    """A mask_mod that is not a band (here: causal inside documents of 200 tokens; and a pattern with holes) and does not
    use the batch or head index: the engine hands its keep matrix and the transpose to the backward as bits
    (ATTN_B200_MASK_BITS) and both launches mask element by element, as the reference's backward does with any
    mask_mod (attn_tl.py:430-461).  Against autograd over the oracle with the same keep matrix."""
    from examples_b200 import programs
    B, H, S, D = 1, 2, 700, 128
    if which == "document":
        mask_mod = lambda b, h, q_idx, kv_idx: torch.logical_and(q_idx >= kv_idx, (q_idx // 200) == (kv_idx // 200))  # noqa: E731
    else:
        mask_mod = lambda b, h, q_idx, kv_idx: torch.logical_or(q_idx == kv_idx, ((q_idx // 64) + (kv_idx // 96)) % 3 == 0)  # noqa: E731
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 61)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(62)).to(torch.bfloat16)
    qi, ki = torch.arange(S)[:, None], torch.arange(S)[None, :]
    keep = mask_mod(0, 0, qi, ki)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        ref = rm.softmax_attention(qf, kf, vf, False, D ** -0.5, keep=keep)
        ref.backward(d_o.float())
    eng = programs.masked_softmax_engine(B, H, S, D, D, mask_mod)
    assert eng._sparse_host is not None and "bits_q" in eng._sparse_host
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), ref.detach(), "o")
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        check(got, want, what)


def test_elementwise_program_under_a_general_mask():
    """relu attention (no online_func) with causal documents of 150 tokens: the derived backward functor with keep bits."""
    from attn_engine import AttentionEngine
    from core import CustomIO, meta_tensor
    B, H, S, D = 1, 2, 500, 64
    scale = D ** -0.5
    mask_mod = lambda b, h, q_idx, kv_idx: torch.logical_and(q_idx >= kv_idx, (q_idx // 150) == (kv_idx // 150))  # noqa: E731
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 71, k_scale=0.5, v_scale=0.5)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(72)).to(torch.bfloat16)
    keep = mask_mod(0, 0, torch.arange(S)[:, None], torch.arange(S)[None, :])
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        s = torch.einsum("bshd,bthd->bhst", qf, kf) * scale
        ref = torch.einsum("bhst,bthd->bshd", torch.relu(s) * keep, vf)
        ref.backward(d_o.float())
    meta = (meta_tensor(B, H, S, D, dtype=torch.bfloat16),) * 3
    eng = AttentionEngine(meta, CustomIO({}), score_mod=lambda sc, c, b, h, qq, kk: (sc * scale).max(0), mask_mod=mask_mod,
                          online_func=None)   # mask_value "-inf": relu(-inf) = 0 (with "0" the forward masks nothing, as the reference)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), ref.detach(), "o")
    for got, want, what in zip((qc.grad, kc.grad, vc.grad), (qf.grad, kf.grad, vf.grad), ("dq", "dk", "dv")):
        check(got, want, what)
