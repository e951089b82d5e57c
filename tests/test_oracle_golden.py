"""The oracle (oracle/reference_math.py) against the committed outputs of the
reference's own PyTorch reference closures (tests/golden/*.pt, produced by
tests/golden/make_golden.py)."""

import math
import os

import pytest
import torch

from oracle import inputs, reference_math as rm

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return torch.load(os.path.join(GOLD, f"{name}.pt"))


def close(a, b, tol=2e-5):
    assert a.shape == b.shape
    err = (a.float() - b.float()).abs().max().item()
    assert err <= tol, f"max abs err {err}"


@pytest.mark.parametrize("name", ["softmax_c1", "softmax_causal_small", "softmax_noncausal_d64"])
def test_softmax(name):
    g = load(name)
    B, H, S, D, Dv = g["shape"]
    dt = torch.float32 if "float32" in g["dtype"] else torch.bfloat16
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"], dtype=dt)
    close(rm.softmax_attention(q, k, v, causal=g["causal"], softmax_scale=D ** -0.5), g["o"])


@pytest.mark.parametrize("name", ["softmax_bwd_causal", "softmax_bwd_noncausal"])
def test_softmax_gradients(name):
    """Gradients through the oracle's closure against autograd through the reference's own (testing/test.py:79-127)."""
    g = load(name)
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"])
    close(rm.softmax_attention(q, k, v, causal=g["causal"], softmax_scale=D ** -0.5), g["o"])
    dq, dk, dv = rm.softmax_attention_grads(q, k, v, g["d_o"], causal=g["causal"], softmax_scale=D ** -0.5)
    close(dq, g["dq"])
    close(dk, g["dk"])
    close(dv, g["dv"])


def test_retention_gradients():
    """Autograd through the oracle's retention closure, and the closed form of the decayed linear attention, against
    autograd through the reference's own closure (testing/test.py:738-770)."""
    g = load("retention_bwd")
    B, H, S, Dk, Dv = g["shape"]
    q, k, v, decay = inputs.retention_bhsd(B, H, S, Dk, Dv, g["seed"])
    close(rm.retention_recurrent(q, k, v), g["o"], tol=2e-4)
    for got, want in zip(rm.retention_grads(q, k, v, g["d_o"]), (g["dq"], g["dk"], g["dv"])):
        close(got, want, tol=2e-4)
    closed = rm.decayed_linear_attention_grads(q, k, v, decay.log(), g["d_o"], scale=Dk ** -0.5)
    for got, want in zip(closed, (g["dq"], g["dk"], g["dv"])):
        close(got, want, tol=2e-4)


@pytest.mark.parametrize("name", ["sigmoid_causal", "sigmoid_noncausal_scaled"])
def test_sigmoid(name):
    g = load(name)
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"])
    qs = q.float() * D ** -0.5 if g["scaled"] else q.float()
    close(rm.sigmoid_attention(qs, k, v, torch.tensor([g["bias"]]), causal=g["causal"]), g["o"])


def test_relu():
    g = load("relu")
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"], k_scale=0.5, v_scale=0.5)
    close(rm.relu_attention(q, k, v), g["o"])


def test_retention():
    g = load("retention")
    B, H, S, Dk, Dv = g["shape"]
    q, k, v, _ = inputs.retention_bhsd(B, H, S, Dk, Dv, g["seed"])
    close(rm.retention_recurrent(q, k, v), g["o"], tol=1e-4)


def test_mla():
    g = load("mla")
    B, H, S, D, Dv = g["shape"]
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, g["seed"])
    close(rm.mla_decode(q[..., :Dv], q[..., Dv:], kv[..., :Dv], kv[..., Dv:]), g["o"])


def test_lse_consistent_with_softmax():
    """The unpinned lse definition must at least reproduce the pinned output: softmax = exp(s - lse)."""
    q, k, v = inputs.attention_bshd(1, 2, 96, 64, 64, 5, dtype=torch.float32)
    lse = rm.softmax_lse(q, k, causal=True)
    s = torch.einsum("bshd,bthd->bhst", q, k) / 8.0
    s = s.masked_fill(~torch.ones(96, 96, dtype=torch.bool).tril(), float("-inf"))
    o = torch.einsum("bhst,bthd->bshd", torch.exp(s - lse[..., None]), v)
    close(o, rm.softmax_attention(q, k, v, causal=True), tol=1e-5)


def test_group_norm_matches_torch():
    x = torch.randn(2, 3, 17, 64, generator=torch.Generator().manual_seed(3))
    want = torch.nn.functional.group_norm(x.permute(0, 2, 1, 3).reshape(2 * 17, 3 * 64), 3, eps=1e-5)
    want = want.view(2, 17, 3, 64).permute(0, 2, 1, 3)
    close(rm.group_norm_heads(x), want, tol=1e-5)


def test_gqa_head_grouping():
    """Head (h*g + j) of the query uses kv head h (rearrange '(h g)' of testing/test.py:86-88)."""
    g = torch.Generator().manual_seed(9)
    q = torch.randn(1, 32, 4, 16, generator=g)
    k = torch.randn(1, 32, 2, 16, generator=g)
    v = torch.randn(1, 32, 2, 16, generator=g)
    o = rm.softmax_attention(q, k, v, causal=False)
    for h in range(4):
        single = rm.softmax_attention(q[:, :, h:h + 1], k[:, :, h // 2:h // 2 + 1], v[:, :, h // 2:h // 2 + 1], causal=False)
        close(o[:, :, h:h + 1], single, tol=1e-6)


def test_gated_retention():
    g = load("gla")
    B, H, S, D, Dv = g["shape"]
    q, k, v, gl = inputs.gla_inputs(B, H, S, D, Dv, g["seed"])
    close(rm.decayed_linear_attention(q, k, v, gl, scale=D ** -0.5), g["o"], tol=1e-4)


def test_mamba2_ssd():
    g = load("mamba2")
    B, HQ, HK, HV, S, D, Dv = g["shape"]
    q, k, v, dt, A = inputs.mamba2_inputs(B, HQ, HK, HV, S, D, Dv, g["seed"])
    o = rm.decayed_linear_attention(q, k, v.float() * dt[..., None], dt * A.view(1, HV, 1), scale=1.0)
    close(o, g["o"], tol=1e-4)


def test_mha_decode():
    """testing/test.py:131-148: a few query rows against a longer KV, no mask"""
    g = load("mha_decode")
    B, H, Sq, KV, D, Dv = g["shape"]
    gen = torch.Generator().manual_seed(g["seed"])
    q = torch.randn(B, Sq, H, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, KV, H, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, KV, H, Dv, generator=gen).to(torch.bfloat16)
    close(rm.softmax_attention(q, k, v, causal=False), g["o"])


def sparse_decode_inputs(g):
    B, H, G, S, D, Dv = g["shape"]
    gen = torch.Generator().manual_seed(g["seed"])
    q = torch.randn(B, 1, H, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, S, G, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, S, G, Dv, generator=gen).to(torch.bfloat16)
    return q, k, v


def test_sparse_gqa_decode():
    """testing/test.py:654-694: block mask per (batch, kv head) and ragged cache lengths"""
    g = load("sparse_gqa_decode")
    q, k, v = sparse_decode_inputs(g)
    close(rm.sparse_gqa_decode(q, k, v, g["block_mask"], g["cache_seqlens"], g["block"]), g["o"])
