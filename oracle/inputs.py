"""Seeded synthetic inputs for the parity tests and the benchmark.  TEST
INFRASTRUCTURE (see reference_math.py).  Inputs are drawn on the CPU in fp32
from a seeded generator and then cast, so the CPU oracle and the GPU kernels
see identical bits.  Distributions follow the reference's tests
(testing/test.py: N(0,1) q/k/v; relu K,V scaled by 0.5, :609-610; retention K
scaled, gamma_h = 1 - 2^(-5-h), :752-755; sigmoid bias scalar, :557)."""

from __future__ import annotations

import math

import torch


def _gen(seed: int) -> torch.Generator:
    return torch.Generator().manual_seed(seed)


def randn(shape, seed: int, dtype=torch.float32, scale: float = 1.0) -> torch.Tensor:
    return (torch.randn(*shape, generator=_gen(seed)) * scale).to(dtype)


def attention_bshd(B, H, S, D, Dv, seed, dtype=torch.bfloat16, k_scale=1.0, v_scale=1.0):
    """q,k: [B,S,H,D], v: [B,S,H,Dv]."""
    g = _gen(seed)
    q = torch.randn(B, S, H, D, generator=g).to(dtype)
    k = (torch.randn(B, S, H, D, generator=g) * k_scale).to(dtype)
    v = (torch.randn(B, S, H, Dv, generator=g) * v_scale).to(dtype)
    return q, k, v


def retention_bhsd(B, H, S, Dk, Dv, seed, dtype=torch.bfloat16, k_scale=None):
    """q,k: [B,H,S,Dk], v: [B,H,S,Dv], decay [B,H,S] fp32 holding gamma_h."""
    k_scale = Dk ** -0.5 if k_scale is None else k_scale
    g = _gen(seed)
    q = torch.randn(B, H, S, Dk, generator=g).to(dtype)
    k = (torch.randn(B, H, S, Dk, generator=g) * k_scale).to(dtype)
    v = torch.randn(B, H, S, Dv, generator=g).to(dtype)
    gamma = 1.0 - torch.exp2(-5.0 - torch.arange(H, dtype=torch.float32))
    decay = gamma[None, :, None].expand(B, H, S).contiguous()
    return q, k, v, decay


def mla_inputs(B, H, S, D, Dv, seed, dtype=torch.bfloat16):
    """q [B,1,H,D], latent KV [B,S,1,D] (V = first Dv columns)."""
    g = _gen(seed)
    q = torch.randn(B, 1, H, D, generator=g).to(dtype)
    kv = torch.randn(B, S, 1, D, generator=g).to(dtype)
    return q, kv


def gla_inputs(B, H, S, D, Dv, seed, dtype=torch.bfloat16):
    """Gated retention / simple GLA (testing/test.py:412-418): q,k [B,H,S,D], v [B,H,S,Dv] N(0,1),
    g [B,H,S] fp32 = logsigmoid(N(0,1)) clamped at -5 (natural-log decay per token)."""
    g_ = _gen(seed)
    q = torch.randn(B, H, S, D, generator=g_).to(dtype)
    k = torch.randn(B, H, S, D, generator=g_).to(dtype)
    v = torch.randn(B, H, S, Dv, generator=g_).to(dtype)
    g = torch.nn.functional.logsigmoid(torch.randn(B, H, S, generator=g_)).clamp_min(-5.0)
    return q, k, v, g


def mamba2_inputs(B, HQ, HK, HV, S, D, Dv, seed, dtype=torch.bfloat16):
    """Mamba2 SSD (testing/test.py:161-180), in the engine's [B,H,S,*] layout: q (= C) [B,HQ,S,D],
    k (= B) [B,HK,S,D] scaled 0.5, v (= x) [B,HV,S,Dv], dt [B,HV,S] fp32 = softplus(0.7 U(0,1) + bias_h),
    A [1,HV] = 1.5 U(0,1) - 4."""
    g_ = _gen(seed)
    q = torch.randn(B, HQ, S, D, generator=g_).to(dtype)
    k = (0.5 * torch.randn(B, HK, S, D, generator=g_)).to(dtype)
    v = torch.randn(B, HV, S, Dv, generator=g_).to(dtype)
    A = (1.5 * torch.rand(HV, generator=g_) - 4.0).to(dtype).float().view(1, HV)
    dt0 = torch.exp(torch.rand(HV, generator=g_) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp(min=1e-4)
    bias = dt0 + torch.log(-torch.expm1(-dt0))
    dt = torch.nn.functional.softplus(0.7 * torch.rand(B, HV, S, generator=g_) + bias.view(1, HV, 1))
    return q, k, v, dt, A


# The five benchmark configurations (shapes, seeds, constants).
CONFIGS = {
    "C1": dict(kind="softmax", B=1, H=4, S=512, D=64, Dv=64, causal=False, seed=1001),
    "C2": dict(kind="softmax", B=8, H=32, S=4096, D=128, Dv=128, causal=True, seed=1002),
    "C3": dict(kind="sigmoid", B=8, H=32, S=4096, D=128, Dv=128, causal=False, seed=1003,
               bias=-math.log(4096.0)),
    "C4": dict(kind="retention", B=8, H=8, S=4096, D=256, Dv=512, chunk=64, seed=1004),
    "C5": dict(kind="mla", B=128, H=128, S=8192, D=576, Dv=512, seed=1005),
}
