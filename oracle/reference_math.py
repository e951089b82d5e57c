"""CPU oracle: a plain fp32 PyTorch restatement of the reference math of the
hot path.  TEST INFRASTRUCTURE ONLY -- imported by tests/, by
__graft_entry__.smoke() and by the CPU-baseline legs of bench.py; the product
(metaattention_b200/) never imports it.

Each function restates one of the inline reference closures of the
reference's functional suite (testing/test.py) in our own code.  Parity
pinning: the reference stores no golden vectors (its tests draw unseeded
random inputs), so the oracle is pinned against outputs of the reference's
own closures, extracted from testing/test.py and executed on seeded inputs by
tests/golden/make_golden.py; the resulting fixtures are committed under
tests/golden/ and checked by tests/test_oracle_golden.py (softmax, sigmoid,
relu, retention, MLA, gated retention, Mamba2, MHA decode, block-sparse GQA
decode).  Two items have no reference closure and are therefore "parity
unpinned": the log-sum-exp output of softmax attention (defined only by
examples/mha.py:64-71) and the per-head group normalisation of the retention
output.
"""

from __future__ import annotations

import math

import torch


def _causal_keep(q_len: int, kv_len: int) -> torch.Tensor:
    return torch.ones(q_len, kv_len, dtype=torch.bool).tril()


def softmax_attention(q, k, v, causal: bool = True, softmax_scale: float | None = None, keep=None):
    """testing/test.py:79-104.  q,k: [B,S,H,D], v: [B,S,Hkv,Dv] with H a multiple of
    Hkv; returns [B,S,H,Dv] fp32.  The mask is applied before the scale.  ``keep`` (bool
    [q_len, kv_len]) replaces the causal mask by an arbitrary one (the reference closure masks with
    -inf the same way, testing/test.py:93-97)."""
    q, k, v = q.float(), k.float(), v.float()
    B, Sq, H, D = q.shape
    Hkv = k.shape[2]
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    g = H // Hkv
    # query head (h*g + j) uses kv head h
    qg = q.view(B, Sq, Hkv, g, D)
    s = torch.einsum("bshgd,bthd->bhgst", qg, k)
    if keep is not None:
        s = s.masked_fill(~keep, float("-inf"))
    elif causal:
        s = s.masked_fill(~_causal_keep(Sq, k.shape[1]), float("-inf"))
    p = torch.softmax(s * scale, dim=-1)
    o = torch.einsum("bhgst,bthd->bshgd", p, v)
    return o.reshape(B, Sq, H, v.shape[-1])


def softmax_attention_grads(q, k, v, d_o, causal: bool = True, softmax_scale: float | None = None):
    """(dq, dk, dv) fp32 of ``softmax_attention`` for the output gradient ``d_o``: torch autograd through the
    restated closure, the way the reference's test obtains the gradients it compares its backward kernels with
    (testing/test.py:106-127)."""
    with torch.enable_grad():
        qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
        o = softmax_attention(qf, kf, vf, causal, softmax_scale)
        o.backward(d_o.float())
    return qf.grad, kf.grad, vf.grad


def softmax_lse(q, k, causal: bool = True, softmax_scale: float | None = None):
    """Per-row log-sum-exp of the scaled, masked scores: [B,H,S] fp32.  No reference
    closure returns it; the definition is the final row scale of examples/mha.py:64-71
    (lse = log(r) + m over the scaled scores).  PARITY UNPINNED."""
    q, k = q.float(), k.float()
    D = q.shape[-1]
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    s = torch.einsum("bshd,bthd->bhst", q, k) * scale
    if causal:
        s = s.masked_fill(~_causal_keep(q.shape[1], k.shape[1]), float("-inf"))
    return torch.logsumexp(s, dim=-1)


def sigmoid_attention(q, k, v, sigmoid_bias, causal: bool = True):
    """testing/test.py:519-543: sigmoid(q.k + bias) written as (tanh(x/2)+1)/2, no
    softmax scale, masked positions give 0.  BSHD in, [B,S,H,Dv] fp32 out."""
    q, k, v = q.float(), k.float(), v.float()
    s = torch.einsum("bshd,bthd->bhst", q, k)
    if causal:
        s = s.masked_fill(~_causal_keep(q.shape[1], k.shape[1]), float("-inf"))
    s = s + torch.as_tensor(sigmoid_bias, dtype=torch.float32)
    p = (torch.tanh(s * 0.5) + 1.0) * 0.5
    return torch.einsum("bhst,bthd->bshd", p, v)


def relu_attention(q, k, v):
    """testing/test.py:599-604: relu(q.k / sqrt(D)) . v, non-causal.  BSHD."""
    q, k, v = q.float(), k.float(), v.float()
    s = torch.einsum("bshd,bthd->bhst", q, k) / math.sqrt(q.shape[-1])
    return torch.einsum("bhst,bthd->bshd", torch.relu(s), v)


def retnet_decay(n_heads: int) -> torch.Tensor:
    """gamma_h = 1 - 2^(-5-h) (testing/test.py:753-755)."""
    return 1.0 - torch.exp2(-5.0 - torch.arange(n_heads, dtype=torch.float32))


def retention_recurrent(q, k, v):
    """testing/test.py:738-747: o[i] = sum_{j<=i} gamma_h^(i-j) (q_i/sqrt(Dk) . k_j) v_j.
    q,k: [B,H,S,Dk], v: [B,H,S,Dv]; returns fp32 [B,H,S,Dv] (the reference casts back
    to the input dtype; the oracle keeps fp32)."""
    q, k, v = q.float(), k.float(), v.float()
    B, H, S, Dk = q.shape
    log2_gamma = torch.log2(retnet_decay(H))
    pos = torch.arange(S, dtype=torch.float32)
    delta = pos.view(-1, 1) - pos.view(1, -1)
    o = torch.empty(B, H, S, v.shape[-1])
    for h in range(H):  # one head at a time keeps the [S,S] decay matrix small
        # The reference multiplies exp2((i-j) log2 gamma) by the 0/1 mask AFTER exponentiating, which
        # gives inf * 0 = NaN once (S-1) |log2 gamma| > 128 (S >= ~2800 for head 0); masking the
        # exponent first is the same function wherever the reference is finite.
        decay = torch.exp2(delta.clamp_min(0.0) * log2_gamma[h]) * (delta >= 0)
        s = torch.einsum("bqd,bkd->bqk", q[:, h] * Dk ** -0.5, k[:, h]) * decay
        o[:, h] = torch.einsum("bqk,bkd->bqd", s, v[:, h])
    return o


def retention_grads(q, k, v, d_o):
    """(dq, dk, dv) fp32 of ``retention_recurrent`` for the output gradient ``d_o``: torch autograd through the
    restated closure (the reference's test differentiates its own closure the same way, testing/test.py:749-770)."""
    with torch.enable_grad():
        qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
        retention_recurrent(qf, kf, vf).backward(d_o.float())
    return qf.grad, kf.grad, vf.grad


def decayed_linear_attention_grads(q, k, v, log_decay, d_o, scale: float = 1.0, with_decay: bool = False):
    """(dq, dk, dv) fp32 of ``decayed_linear_attention``, in closed form with the decay matrix D_ij = exp(G_i - G_j),
    j <= i, in fp64: dq = scale (D o (dO V^T)) K, dk = scale (D o (dO V^T))^T Q, dv = scale (D o (Q K^T))^T dO.  Heads of
    q / k shared by several heads of v get the sum of their gradients.  ``with_decay``: a fourth result, the gradient
    with respect to ``log_decay`` (its shape), by torch autograd through the matrix form o = scale (D o Q K^T) V — how the
    reference's test obtains the gradients it compares its kernels with (testing/test.py:106-127)."""
    q, k, v, ld, d_o = q.double(), k.double(), v.double(), log_decay.double(), d_o.double()
    B, H, S, _ = v.shape
    HQ, HK = q.shape[1], k.shape[1]
    qe = q.repeat_interleave(H // HQ, dim=1)
    ke = k.repeat_interleave(H // HK, dim=1)
    tril = torch.ones(S, S, dtype=torch.float64).tril()
    G = ld.expand(B, H, S).cumsum(-1)
    D = torch.exp((G.unsqueeze(-1) - G.unsqueeze(-2)).clamp_max(0.0)) * tril
    a = D * torch.einsum("bhid,bhjd->bhij", d_o, v) * scale
    dq = torch.einsum("bhij,bhjd->bhid", a, ke)
    dk = torch.einsum("bhij,bhid->bhjd", a, qe)
    dv = torch.einsum("bhij,bhid->bhjd", D * torch.einsum("bhid,bhjd->bhij", qe, ke) * scale, d_o)
    dq = dq.view(B, HQ, H // HQ, S, -1).sum(2)
    dk = dk.view(B, HK, H // HK, S, -1).sum(2)
    if not with_decay:
        return dq.float(), dk.float(), dv.float()
    with torch.enable_grad():
        ldv = ld.clone().requires_grad_(True)
        Gv = ldv.expand(B, H, S).cumsum(-1)
        # masked before the exponential: above the diagonal the exponent is positive and may overflow
        Dv_ = torch.exp((Gv.unsqueeze(-1) - Gv.unsqueeze(-2)).masked_fill(tril == 0, float("-inf")))
        o = torch.einsum("bhij,bhjd->bhid", Dv_ * torch.einsum("bhid,bhjd->bhij", qe, ke) * scale, v)
        (dld,) = torch.autograd.grad(o, ldv, d_o)
    return dq.float(), dk.float(), dv.float(), dld.float()


def decayed_linear_attention(q, k, v, log_decay, scale: float = 1.0):
    """o[i] = sum_{j<=i} exp(G_i - G_j) (scale q_i . k_j) v_j with G the inclusive cumulative sum of the
    per-token natural-log decay: the function computed chunk by chunk by naive_chunk_simple_gla
    (testing/test.py:436-481, gated retention, scale = 1/sqrt(D)) and by ssd_chunk_scan_combined_ref
    (testing/test.py:305-343, Mamba2 SSD with q = C, k = B, v = x dt, log_decay = dt A, scale = 1).
    q [B,HQ,S,D] and k [B,HK,S,D] may have fewer heads than v [B,H,S,Dv]: head h of v uses group
    h // (H / HQ) (the SSD reference repeats each group consecutively, testing/test.py:222,271).
    Evaluated as a plain token recurrence over the state in fp64; returns fp32 [B,H,S,Dv]."""
    q, k, v, log_decay = q.double(), k.double(), v.double(), log_decay.double()
    B, H, S, Dv = v.shape
    if q.shape[1] != H:
        q = q.repeat_interleave(H // q.shape[1], dim=1)
    if k.shape[1] != H:
        k = k.repeat_interleave(H // k.shape[1], dim=1)
    state = torch.zeros(B, H, q.shape[-1], Dv, dtype=torch.float64)
    o = torch.empty(B, H, S, Dv, dtype=torch.float64)
    for i in range(S):
        state = state * torch.exp(log_decay[:, :, i])[..., None, None] + k[:, :, i, :, None] * v[:, :, i, None, :]
        o[:, :, i] = torch.einsum("bhd,bhde->bhe", q[:, :, i] * scale, state)
    return o.float()


def group_norm_heads(o, eps: float = 1e-5):
    """Normalisation of each (batch, head, token) vector over Dv to zero mean and unit
    variance, no affine parameters (GroupNorm with one group per head).  The reference
    has no such step anywhere; PARITY UNPINNED."""
    o = o.float()
    mean = o.mean(dim=-1, keepdim=True)
    var = o.var(dim=-1, unbiased=False, keepdim=True)
    return (o - mean) * torch.rsqrt(var + eps)


def retention_parallel(q, k, v, mask):
    """attention_engine/benchmark/bench_utils.py:1158-1163: s = (q.k) * mask,
    o = (s / clamp(sum|s|, min=1)) . v.  q,k,v: [B,S,H,*], mask: [1,H,S,S]."""
    q, k, v, mask = q.float(), k.float(), v.float(), mask.float()
    s = torch.einsum("bshd,bthd->bhst", q, k) * mask
    s = s / s.abs().sum(dim=-1, keepdim=True).clamp(min=1.0)
    return torch.einsum("bhst,bthd->bshd", s, v)


def mla_decode(q, q_pe, kv, k_pe):
    """testing/test.py:807-839: one query token per sequence attends to a shared latent KV
    head.  q: [B,1,H,Dv], q_pe: [B,1,H,Dr], kv: [B,S,Hkv,Dv], k_pe: [B,S,Hkv,Dr];
    score = ([q,q_pe] . [kv,k_pe]) / sqrt(Dv+Dr); out = softmax . kv -> [B,1,H,Dv] fp32."""
    q, q_pe, kv, k_pe = q.float(), q_pe.float(), kv.float(), k_pe.float()
    B, _, H, Dv = q.shape
    Hkv = kv.shape[2]
    g = H // Hkv
    query = torch.cat([q[:, 0], q_pe[:, 0]], dim=-1).view(B, Hkv, g, -1)   # head (h*g+j) uses kv head h
    key = torch.cat([kv, k_pe], dim=-1)
    s = torch.einsum("bhgd,bshd->bhgs", query, key) / math.sqrt(query.shape[-1])
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("bhgs,bshd->bhgd", p, kv)
    return o.reshape(B, 1, H, Dv)


def mla_decode_lse(q, q_pe, kv, k_pe):
    """Natural-log sum-exp of the scaled scores, [B,H] fp32 (what the reference's native
    MLA path returns as softmax_lse, cute_template_kvshared/flash_mla_interface.py:98-115).
    No reference closure computes it; PARITY UNPINNED."""
    q, q_pe, kv, k_pe = q.float(), q_pe.float(), kv.float(), k_pe.float()
    B, _, H, _ = q.shape
    Hkv = kv.shape[2]
    g = H // Hkv
    query = torch.cat([q[:, 0], q_pe[:, 0]], dim=-1).view(B, Hkv, g, -1)
    key = torch.cat([kv, k_pe], dim=-1)
    s = torch.einsum("bhgd,bshd->bhgs", query, key) / math.sqrt(query.shape[-1])
    return torch.logsumexp(s, dim=-1).reshape(B, H)


def sparse_gqa_decode(q, k, v, block_mask, cache_seqlens, block_size: int):
    """testing/test.py:654-694 (``ref_program_torch``): one query token per sequence, grouped KV heads, only
    the KV blocks flagged in ``block_mask`` [B, Hkv, blocks] and the first ``cache_seqlens[b]`` positions take
    part in the softmax; scale 1/sqrt(D).  q: [B,1,H,D], k: [B,S,Hkv,D], v: [B,S,Hkv,Dv]; query head
    (h*g + j) uses KV head h.  Returns [B,H,Dv] fp32."""
    q, k, v = q.float(), k.float(), v.float()
    B, _, H, D = q.shape
    S, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    keep = block_mask.bool().repeat_interleave(block_size, dim=-1)[..., :S]            # [B, Hkv, S]
    if keep.shape[-1] < S:
        keep = torch.nn.functional.pad(keep, (0, S - keep.shape[-1]))
    keep = keep & (torch.arange(S).view(1, 1, S) < cache_seqlens.view(B, 1, 1))
    s = torch.einsum("bhgd,bshd->bhgs", q[:, 0].view(B, Hkv, g, D), k) / math.sqrt(D)
    s = s.masked_fill(~keep[:, :, None, :], float("-inf"))
    o = torch.einsum("bhgs,bshd->bhgd", torch.softmax(s, dim=-1), v)
    return o.reshape(B, H, v.shape[-1])
