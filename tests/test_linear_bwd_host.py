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

    def fake_forward(q, k, v, log_decay, q_scale=1.0, normalize=False, eps=1e-5, out_dtype=None):
        assert q.shape[-1] in (64, 128, 256), "the kernel covers these widths of dim_qk only"
        assert not normalize
        return rm.decayed_linear_attention(q, k, v, log_decay, scale=q_scale)

    monkeypatch.setattr(le, "linear_attention_forward", fake_forward)
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
