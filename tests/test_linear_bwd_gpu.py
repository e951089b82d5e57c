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


def test_programs_with_operand_mods_say_so():
    """Mamba2's v_mod rewrites v before the kernel: its derivative is not built."""
    from examples_b200 import programs
    B, HQ, HK, HV, S, D, Dv = 1, 2, 2, 4, 128, 64, 64
    q, k, v, dt, A = inputs.mamba2_inputs(B, HQ, HK, HV, S, D, Dv, 71)
    eng = programs.mamba2_engine(B, HQ, S, D, Dv, HK=HK, HV=HV)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = eng(qc, kc, vc, dt.cuda(), A.cuda(), dt.to(torch.bfloat16).cuda())
    with pytest.raises(NotImplementedError):
        o.sum().backward()
