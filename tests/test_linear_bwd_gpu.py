"""Backward of chunked linear attention / retention (``linear_attention_backward`` and the engine's autograd path:
five runs of the forward kernel) against the committed gradients of the reference's own retention closure
(tests/golden/retention_bwd.pt: torch autograd through testing/test.py:738-747) and against the oracle's closed form
on further shapes.  16-bit results against fp32: max-abs 2e-2 and mean-abs 3e-3, each scaled by the magnitude of the
expected tensor where that exceeds 1 (its largest value for the maximum, its standard deviation for the mean):
gradients of slowly decaying heads sum over hundreds of tokens and reach magnitudes of 10 to 70, and rounding a
result of standard deviation s to bf16 costs a mean-abs error of 2.2e-3 s by itself (measured: every head of every
shape below sits at 2.17-2.23e-3 s, maximum 3-5e-3 of the largest value)."""

import os

import pytest
import torch

from oracle import inputs, reference_math as rm

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def check(got, want, what):
    d = (got.float().cpu() - want.float()).abs()
    assert torch.isfinite(got).all(), what
    assert d.max().item() <= 2e-2 * max(1.0, want.abs().max().item()), (what, d.max().item(), want.abs().max().item())
    assert d.mean().item() <= 3e-3 * max(1.0, want.std().item()), (what, d.mean().item(), want.std().item())


def check_decay_grad(got, want, what):
    """Gradients that pass through the log-decays: dg_t is a reversed running sum over the tokens of q_i . dq_i -
    k_i . dk_i, a difference of two sums whose 16-bit rounding errors (the kernel rounds its decayed scores to 16 bits)
    then add up along the sequence like a random walk; the runs it is formed from therefore keep a 16-bit remainder
    of those scores (``precise``).  The reference's test means to hold g.grad to rtol 3e-2 (testing/test.py:513-518,
    switched off there); here: mean-abs 3e-2 of the expected spread, max-abs 1e-1 of the largest value (measured: dg
    mean-abs 2.3e-3 of the spread, Mamba2's dA, a sum over all tokens, 2.7e-2; without the remainder dg had 1.2e-2 and dA
    9e-2)."""
    d = (got.float().cpu() - want.float()).abs()
    assert torch.isfinite(got).all(), what
    assert d.max().item() <= 1e-1 * max(1.0, want.abs().max().item()), (what, d.max().item(), want.abs().max().item())
    assert d.mean().item() <= 3e-2 * max(1.0, want.std().item()), (what, d.mean().item(), want.std().item())


def test_against_reference_golden():
    from examples_b200 import programs
    g = torch.load(os.path.join(GOLD, "retention_bwd.pt"))
    B, H, S, Dk, Dv = g["shape"]
    q, k, v, decay = inputs.retention_bhsd(B, H, S, Dk, Dv, g["seed"])
    eng = programs.retnet_engine(B, H, S, Dk, Dv)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc, decay.cuda())
    o.backward(g["d_o"].cuda())
    torch.cuda.synchronize()
    check(o.detach(), g["o"], "o")
    check(qc.grad, g["dq"], "dq")
    check(kc.grad, g["dk"], "dk")
    check(vc.grad, g["dv"], "dv")


@pytest.mark.parametrize("B,H,S,Dk,Dv", [
    (1, 4, 512, 256, 512),    # the benchmark's head dims: contractions over dim_v = 512 run as two halves
    (2, 2, 300, 64, 128),     # ragged last block
    (1, 2, 200, 128, 384),    # dim_v = 256 + 128
])
def test_retention_shapes_against_oracle(B, H, S, Dk, Dv):
    from attn_engine.linear_attn_engine import linear_attention_backward
    q, k, v, decay = inputs.retention_bhsd(B, H, S, Dk, Dv, S + Dk)
    d_o = torch.randn(B, H, S, Dv, generator=torch.Generator().manual_seed(S)).to(torch.bfloat16)
    want = rm.decayed_linear_attention_grads(q, k, v, decay.log(), d_o, scale=Dk ** -0.5)
    got = linear_attention_backward(q.cuda(), k.cuda(), v.cuda(), decay.log().cuda(), d_o.cuda(), q_scale=Dk ** -0.5)
    torch.cuda.synchronize()
    for g_, w_, what in zip(got, want, ("dq", "dk", "dv")):
        check(g_, w_, what)


def test_gated_retention_per_token_decay():
    """Per-token log-decays (gated retention, examples/gated_retention.py): the time-reversed runs take the decays
    shifted by one token."""
    from examples_b200 import programs
    B, H, S, D, Dv = 1, 4, 200, 64, 128
    q, k, v, g = inputs.gla_inputs(B, H, S, D, Dv, 61)
    d_o = torch.randn(B, H, S, Dv, generator=torch.Generator().manual_seed(62)).to(q.dtype)
    want = rm.decayed_linear_attention_grads(q, k, v, g, d_o, scale=D ** -0.5)
    eng = programs.gla_engine(B, H, S, D, Dv)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc, g.cuda())
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    check(o.detach(), rm.decayed_linear_attention(q, k, v, g, scale=D ** -0.5), "o")
    for got, w_, what in zip((qc.grad, kc.grad, vc.grad), want, ("dq", "dk", "dv")):
        check(got, w_, what)


def test_gated_retention_gradient_of_the_gates():
    """A learned gate: the per-token log-decay requires grad, and its gradient (reversed sum of q . dq - k . dk) comes
    back with dq, dk, dv; against torch autograd through the oracle's matrix form."""
    from examples_b200 import programs
    B, H, S, D, Dv = 1, 4, 300, 64, 128
    q, k, v, g = inputs.gla_inputs(B, H, S, D, Dv, 63)
    d_o = torch.randn(B, H, S, Dv, generator=torch.Generator().manual_seed(64)).to(q.dtype)
    want = rm.decayed_linear_attention_grads(q, k, v, g, d_o, scale=D ** -0.5, with_decay=True)
    eng = programs.gla_engine(B, H, S, D, Dv)
    qc, kc, vc, gc = (t.cuda().requires_grad_() for t in (q, k, v, g))
    o = eng(qc, kc, vc, gc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    for got, w_, what in zip((qc.grad, kc.grad, vc.grad, gc.grad), want, ("dq", "dk", "dv", "dg")):
        assert got is not None and got.shape == w_.shape, what
        (check_decay_grad if what == "dg" else check)(got, w_, what)


def test_mamba2_gradients_through_the_mods():
    """Mamba2 (v_mod = v * dt, decay_mod = dt * A, grouped q / k heads): gradients of q, k, v and of the custom inputs dt
    and A, against autograd over the same program in fp64 torch operations (the matrix form of testing/test.py:305-343)."""
    from examples_b200 import programs
    B, HQ, HK, HV, S, D, Dv = 1, 2, 2, 4, 256, 64, 128
    q, k, v, dt, A = inputs.mamba2_inputs(B, HQ, HK, HV, S, D, Dv, 71)
    d_o = torch.randn(B, HV, S, Dv, generator=torch.Generator().manual_seed(72)).to(q.dtype)
    eng = programs.mamba2_engine(B, HQ, S, D, Dv, HK=HK, HV=HV)
    leaves = [t.cuda().requires_grad_() for t in (q, k, v, dt, A)]
    qc, kc, vc, dtc, Ac = leaves
    o = eng(qc, kc, vc, dtc, Ac, dtc)
    o.backward(d_o.cuda())
    torch.cuda.synchronize()
    ref = [t.clone().double().requires_grad_() for t in (q, k, v, dt, A)]
    qr, kr, vr, dtr, Ar = ref
    ld = dtr * Ar.view(1, -1, 1)
    vv = vr * dtr.unsqueeze(-1)
    G = ld.cumsum(-1)
    tril = torch.ones(S, S, dtype=torch.float64).tril()
    Dm = torch.exp((G.unsqueeze(-1) - G.unsqueeze(-2)).masked_fill(tril == 0, float("-inf")))
    qe, ke = qr.repeat_interleave(HV // HQ, dim=1), kr.repeat_interleave(HV // HK, dim=1)
    o_ref = torch.einsum("bhij,bhjd->bhid", Dm * torch.einsum("bhid,bhjd->bhij", qe, ke), vv)
    check(o.detach(), o_ref.detach().float(), "o")
    o_ref.backward(d_o.double())
    for got, want, what in zip(leaves, ref, ("dq", "dk", "dv", "d dt", "dA")):
        assert got.grad is not None, what
        (check_decay_grad if what in ("d dt", "dA") else check)(got.grad, want.grad.float(), what)


def test_normalised_output_says_so():
    """The output normalisation of the retention benchmark has no backward: differentiating it is refused."""
    from examples_b200 import programs
    B, H, S, Dk, Dv = 1, 2, 128, 64, 128
    q, k, v, decay = inputs.retention_bhsd(B, H, S, Dk, Dv, 5)
    eng = programs.retnet_engine(B, H, S, Dk, Dv)
    eng.normalize_output = True
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc, decay.cuda())
    with pytest.raises(NotImplementedError):
        o.float().sum().backward()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_row_kernels_against_torch(dtype):
    """The reversed / column-sliced copy and the sum + cast + reversal of partial results, bit for bit against torch."""
    from core.native import lib
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 301, 384, generator=g).to(dtype).cuda()
    for col0, width, rev in [(0, 384, True), (128, 256, True), (256, 128, False), (8, 24, True)]:
        got = lib.rows_copy(x, col0, width, rev)
        want = x[..., col0:col0 + width]
        want = (want.flip(2) if rev else want).contiguous()
        assert got.is_contiguous() and torch.equal(got, want), (col0, width, rev)
    a = torch.randn(2, 3, 301, 256, generator=g).cuda()
    b = torch.randn(2, 3, 301, 256, generator=g).cuda()
    for second, rev in [(b, True), (None, True), (b, False)]:
        got = lib.rows_sum_cast(a, second, dtype, rev)
        want = (a if second is None else a + second).to(dtype)
        assert torch.equal(got, want.flip(2) if rev else want), (second is None, rev)
    with pytest.raises(lib.NativeError):
        lib.rows_copy(x, 4, 16, True)      # offsets and widths in units of 8 columns (16 bytes)
