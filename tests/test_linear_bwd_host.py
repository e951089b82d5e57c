"""Host logic of the linear-attention backward without a GPU: ``linear_attention_backward`` composes the gradients
from runs of the forward kernel (time reversals, shifted decays, contractions split by column range, gradients of
shared heads added up).  Here the kernel is replaced by the oracle's decayed linear attention, so that the
composition itself is checked against the closed-form gradients on the CPU."""

import pytest
import torch

from oracle import inputs, reference_math as rm


@pytest.fixture
def oracle_kernel(monkeypatch):
    from attn_engine import linear_attn_engine as le

    def fake_forward(q, k, v, log_decay, q_scale=1.0, normalize=False, eps=1e-5, out_dtype=None, v_scale=None, precise=False):
        assert v_scale is None
        assert q.shape[-1] in (64, 128, 256), "the kernel covers these widths of dim_qk only"
        assert not normalize
        return rm.decayed_linear_attention(q, k, v, log_decay, scale=q_scale)

    def fake_rows_copy(src, col0=0, width=None, reverse=False):
        part = src[..., col0:col0 + (src.shape[-1] - col0 if width is None else width)]
        return (part.flip(-2) if reverse else part).contiguous()

    def fake_rows_sum_cast(a, b, dtype, reverse=False):
        out = (a if b is None else a + b).to(dtype)
        return out.flip(-2) if reverse else out

    monkeypatch.setattr(le, "linear_attention_forward", fake_forward)
    monkeypatch.setattr(le.native, "rows_copy", fake_rows_copy)
    monkeypatch.setattr(le.native, "rows_sum_cast", fake_rows_sum_cast)
    return le


@pytest.mark.parametrize("B,H,S,Dk,Dv", [(1, 2, 96, 64, 128), (1, 2, 70, 64, 320), (2, 1, 50, 128, 600)])
def test_composition_matches_closed_form(oracle_kernel, B, H, S, Dk, Dv):
    g = torch.Generator().manual_seed(S)
    q = torch.randn(B, H, S, Dk, generator=g)
    k = torch.randn(B, H, S, Dk, generator=g) * Dk ** -0.5
    v = torch.randn(B, H, S, Dv, generator=g)
    d_o = torch.randn(B, H, S, Dv, generator=g)
    log_decay = -torch.rand(B, H, S, generator=g) * 0.2          # per-token decays: the reversed runs shift them
    want = rm.decayed_linear_attention_grads(q, k, v, log_decay, d_o, scale=0.37)
    got = oracle_kernel.linear_attention_backward(q, k, v, log_decay, d_o, q_scale=0.37)
    for a, b, what in zip(got, want, ("dq", "dk", "dv")):
        assert a.shape == b.shape, what
        assert (a - b).abs().max().item() <= 2e-4 * max(1.0, b.abs().max().item()), (what, (a - b).abs().max().item())


def test_constant_decay_is_symmetric_under_reversal(oracle_kernel):
    """RetNet: one decay per head; the shifted, reversed decay row differs from the original only in its first entry,
    which no product uses."""
    B, H, S, Dk, Dv = 1, 3, 64, 64, 128
    q, k, v, decay = inputs.retention_bhsd(B, H, S, Dk, Dv, 5)
    d_o = torch.randn(B, H, S, Dv, generator=torch.Generator().manual_seed(6))
    want = rm.decayed_linear_attention_grads(q.float(), k.float(), v.float(), decay.log(), d_o, scale=Dk ** -0.5)
    got = oracle_kernel.linear_attention_backward(q.float(), k.float(), v.float(), decay.log(), d_o, q_scale=Dk ** -0.5)
    for a, b in zip(got, want):
        assert (a - b).abs().max().item() <= 2e-4 * max(1.0, b.abs().max().item())


def test_decay_gradient_is_the_reversed_sum_of_row_minus_column_terms(oracle_kernel):
    """dg_t = sum_{i>=t} (q_i . dq_i - k_i . dk_i) against torch autograd through the matrix form (per-token decays)."""
    B, H, S, Dk, Dv = 2, 2, 80, 64, 128
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, H, S, Dk, generator=g)
    k = torch.randn(B, H, S, Dk, generator=g) * Dk ** -0.5
    v = torch.randn(B, H, S, Dv, generator=g)
    d_o = torch.randn(B, H, S, Dv, generator=g)
    log_decay = -torch.rand(B, H, S, generator=g) * 0.3
    want = rm.decayed_linear_attention_grads(q, k, v, log_decay, d_o, scale=0.5, with_decay=True)
    got = oracle_kernel.linear_attention_backward(q, k, v, log_decay, d_o, q_scale=0.5, need_dg=True)
    assert got[3].shape == (B, H, S)
    for a, b, what in zip(got, want, ("dq", "dk", "dv", "dg")):
        assert (a - b).abs().max().item() <= 3e-4 * max(1.0, b.abs().max().item()), (what, (a - b).abs().max().item())


def test_engine_differentiates_through_its_mods(oracle_kernel):
    """Mamba2 (testing/test.py:305-343 as an engine program: v_mod = v * dt, decay_mod = dt * A, grouped q / k heads):
    gradients of q, k, v and of the custom inputs dt and A arrive through the mods, against autograd over the same
    program written with torch operations around the oracle's matrix form."""
    from examples_b200 import programs
    B, HQ, HK, HV, S, D, Dv = 1, 2, 2, 4, 48, 64, 64
    q, k, v, dt, A = inputs.mamba2_inputs(B, HQ, HK, HV, S, D, Dv, 71)
    q, k, v = q.float(), k.float(), v.float()
    eng = programs.mamba2_engine(B, HQ, S, D, Dv, HK=HK, HV=HV, dtype=torch.float32)
    d_o = torch.randn(B, HV, S, Dv, generator=torch.Generator().manual_seed(72))
    leaves = [t.clone().requires_grad_() for t in (q, k, v, dt, A)]
    qc, kc, vc, dtc, Ac = leaves
    o = eng(qc, kc, vc, dtc, Ac, dtc)
    o.backward(d_o)
    # the same program, every step a torch operation
    ref = [t.clone().double().requires_grad_() for t in (q, k, v, dt, A)]
    qr, kr, vr, dtr, Ar = ref
    ld = dtr * Ar.view(1, -1, 1)
    vv = vr * dtr.unsqueeze(-1)
    G = ld.cumsum(-1)
    tril = torch.ones(S, S, dtype=torch.float64).tril()
    Dm = torch.exp((G.unsqueeze(-1) - G.unsqueeze(-2)).masked_fill(tril == 0, float("-inf")))
    qe, ke = qr.repeat_interleave(HV // HQ, dim=1), kr.repeat_interleave(HV // HK, dim=1)
    o_ref = torch.einsum("bhij,bhjd->bhid", Dm * torch.einsum("bhid,bhjd->bhij", qe, ke), vv)
    assert (o.detach().double() - o_ref.detach()).abs().max().item() <= 1e-3 * max(1.0, o_ref.abs().max().item())
    o_ref.backward(d_o.double())
    for got, want, what in zip(leaves, ref, ("dq", "dk", "dv", "d dt", "dA")):
        assert got.grad is not None, what
        err = (got.grad.double() - want.grad).abs().max().item()
        assert err <= 2e-3 * max(1.0, want.grad.abs().max().item()), (what, err)
