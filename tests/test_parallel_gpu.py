"""Parity of the sm_100a parallel-pattern forward (through the AttentionEngine
API and the C ABI) against the CPU oracle and the committed golden outputs of
the reference's PyTorch closures.

Tolerance (BASELINE north star): 16-bit output against the fp32 reference on
identical seeded inputs, max-abs <= 2e-2 and mean-abs <= 2e-3."""

import math
import os

import pytest
import torch

from examples_b200 import programs
from core.native import lib as native_lib
from oracle import inputs, reference_math as rm

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS = 2e-2, 2e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def check(o, want, max_abs=MAX_ABS, mean_abs=MEAN_ABS):
    from core.native import lib
    assert lib.last_device_status() == 0
    o = o.float().cpu()
    assert not torch.isnan(o).any(), "NaN in output (unwritten rows?)"
    d = (o - want.float()).abs()
    assert d.max().item() <= max_abs and d.mean().item() <= mean_abs, \
        f"max abs {d.max().item():.4g} mean abs {d.mean().item():.4g}"


def cuda(*ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("name", ["softmax_c1", "softmax_causal_small", "softmax_noncausal_d64"])
def test_softmax_against_reference_golden(name):
    g = torch.load(os.path.join(GOLD, f"{name}.pt"))
    B, H, S, D, Dv = g["shape"]
    # golden inputs were fp32 or bf16-rounded; the kernel runs bf16 either way
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"], dtype=torch.bfloat16)
    e = programs.softmax_engine(B, H, S, D, Dv, is_causal=g["causal"])
    o = e(*cuda(q, k, v))
    if "float32" in g["dtype"]:
        # reference ran on the un-rounded fp32 inputs: compare against the oracle on the rounded ones too
        check(o, rm.softmax_attention(q, k, v, g["causal"]))
        check(o, g["o"], max_abs=5e-2, mean_abs=5e-3)
    else:
        check(o, g["o"])


@pytest.mark.parametrize("B,H,S,D,causal,dtype", [
    (1, 4, 512, 64, False, torch.bfloat16),      # BASELINE config 1 semantics
    (2, 3, 1000, 128, True, torch.bfloat16),     # ragged: S not a multiple of the tile
    (1, 2, 77, 64, True, torch.float16),         # shorter than one tile
    (1, 1, 129, 128, False, torch.float16),      # one row into the second tile
    (3, 5, 384, 128, True, torch.float16),       # odd tile count: second query tile of the last CTA is empty
    (1, 2, 2048, 128, True, torch.bfloat16),
])
def test_softmax_shapes_and_lse(B, H, S, D, causal, dtype):
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 100 + S, dtype=dtype)
    e = programs.softmax_engine(B, H, S, D, D, dtype=dtype, is_causal=causal)
    o = e(*cuda(q, k, v))
    check(o, rm.softmax_attention(q, k, v, causal))
    lse = e.last_final_rowscales["lse"].cpu()
    assert (lse - rm.softmax_lse(q, k, causal)).abs().max().item() < 1e-3


def test_guard_bands_untouched_and_strided_views():
    """Outputs are written only inside the logical tensor: q/k/v/o are interior views of
    larger buffers whose surroundings hold NaN canaries (q/k/v) or a sentinel (o)."""
    B, H, S, D = 2, 3, 300, 64
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 7)
    big = [torch.full((B, S + 16, H + 2, D), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(3)]
    views = []
    for buf, t in zip(big, (q, k, v)):
        buf[:, 8:8 + S, 1:1 + H] = t.cuda()
        views.append(buf[:, 8:8 + S, 1:1 + H])
    from core.native import lib
    obuf = torch.full((B, S + 16, H + 2, D), 777.0, dtype=torch.bfloat16, device="cuda")
    o = obuf[:, 8:8 + S, 1:1 + H]
    args = lib.fill_parallel_args(*views, o, mask_kind=lib.MASK_CAUSAL, fparams=[D ** -0.5])
    lib.parallel_fwd(args)
    check(o, rm.softmax_attention(q, k, v, True))
    outside = obuf.clone()
    outside[:, 8:8 + S, 1:1 + H] = 777.0
    assert bool((outside == 777.0).all()), "kernel wrote outside the output view"


def test_generic_lowering_with_rescale_matches_builtin():
    B, H, S, D = 1, 2, 640, 128
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 8)
    e = programs.softmax_engine_noprobe(B, H, S, D, D, is_causal=True)
    assert e.functor_kind == "lowered"
    o = e(*cuda(q, k, v))
    check(o, rm.softmax_attention(q, k, v, True))
    assert (e.last_final_rowscales["lse"].cpu() - rm.softmax_lse(q, k, True)).abs().max().item() < 1e-3
    scaled_max = (torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * D ** -0.5) \
        .masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf")).max(-1).values
    assert (e.last_final_rowscales["rowmax"].cpu() - scaled_max).abs().max().item() < 1e-3


@pytest.mark.parametrize("name", ["sigmoid_causal", "sigmoid_noncausal_scaled"])
def test_sigmoid_against_reference_golden(name):
    g = torch.load(os.path.join(GOLD, f"{name}.pt"))
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"])
    e = programs.sigmoid_engine(B, H, S, D, Dv, is_causal=g["causal"], scale=D ** -0.5 if g["scaled"] else 1.0)
    o = e(*cuda(q, k, v), torch.tensor([g["bias"]], device="cuda"))
    # the reference's own tolerance for sigmoid is 1e-1 (testing/test.py:571); sums of S values in [0,1]
    # times N(0,1) carry bf16 rounding of P, so the un-normalised causal case uses a wider absolute bound
    if g["scaled"]:
        check(o, g["o"])
    else:
        check(o, g["o"], max_abs=1e-1, mean_abs=1e-2)


def test_sigmoid_online_func_none():
    B, H, S, D = 1, 2, 300, 64
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 9)
    bias = torch.tensor([-math.log(S)])
    e = programs.sigmoid_engine(B, H, S, D, D, is_causal=False, scale=D ** -0.5, online=None)
    o = e(*cuda(q, k, v), bias.cuda())
    check(o, rm.sigmoid_attention(q.float() * D ** -0.5, k, v, bias, False))


def test_relu_against_reference_golden():
    g = torch.load(os.path.join(GOLD, "relu.pt"))
    B, H, S, D, Dv = g["shape"]
    q, k, v = inputs.attention_bshd(B, H, S, D, Dv, g["seed"], k_scale=0.5, v_scale=0.5)
    o = programs.relu_engine(B, H, S, D, Dv)(*cuda(q, k, v))
    # outputs are sums of ~S/2 positive weights: scale the tolerance to the reference's own 1e-1 (test.py:623)
    check(o, g["o"], max_abs=1e-1, mean_abs=1e-2)


def test_retention_parallel_custom_tile_input():
    B, H, S, D = 1, 2, 384, 64
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 10)
    mask = torch.rand(1, H, S, S, generator=torch.Generator().manual_seed(2)).tril().to(torch.bfloat16)
    e = programs.retention_parallel_engine(B, H, S, D, D)
    o = e(*cuda(q, k, v, mask))
    check(o, rm.retention_parallel(q, k, v, mask))
    den = (torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * mask.float()).abs().sum(-1).clamp(min=1.0)
    assert ((e.last_final_rowscales["den"].cpu() - den).abs() / den).max().item() < 2e-2


def test_full_size_config2_sampled_heads():
    """BASELINE config 2 (B=8,H=32,S=4096,D=128, causal, bf16 + lse) at full size.  The CPU
    oracle is evaluated on a sample of (batch, head) slices; a checksum over all heads
    guards the rest (every (b, h) slice must be finite and have the right first row: row 0
    attends to key 0 only, so o[b,0,h] == v[b,0,h])."""
    c = inputs.CONFIGS["C2"]
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    q, k, v = inputs.attention_bshd(B, H, S, D, D, c["seed"])
    e = programs.softmax_engine(B, H, S, D, D, is_causal=True)
    o = e(*cuda(q, k, v)).cpu()
    from core.native import lib
    assert lib.last_device_status() == 0
    assert torch.isfinite(o.float()).all()
    assert torch.equal(o[:, 0], v[:, 0])
    lse = e.last_final_rowscales["lse"].cpu()
    for b, h in [(0, 0), (3, 17), (7, 31)]:
        sl = lambda t: t[b:b + 1, :, h:h + 1]
        check(sl(o), rm.softmax_attention(sl(q), sl(k), sl(v), True))
        assert (lse[b, h] - rm.softmax_lse(sl(q), sl(k), True)[0, 0]).abs().max().item() < 1e-3


def test_full_size_config3_sampled_heads():
    """BASELINE config 3: sigmoid(q.k/sqrt(128) - ln 4096), non-causal, full size, sampled heads."""
    c = inputs.CONFIGS["C3"]
    B, H, S, D = c["B"], c["H"], c["S"], c["D"]
    q, k, v = inputs.attention_bshd(B, H, S, D, D, c["seed"])
    bias = torch.tensor([c["bias"]])
    e = programs.sigmoid_engine(B, H, S, D, D, is_causal=False, scale=D ** -0.5)
    o = e(*cuda(q, k, v), bias.cuda()).cpu()
    assert torch.isfinite(o.float()).all()
    for b, h in [(0, 0), (5, 9)]:
        sl = lambda t: t[b:b + 1, :, h:h + 1]
        check(sl(o), rm.sigmoid_attention(sl(q).float() * D ** -0.5, sl(k), sl(v), bias, False))


def test_backward_is_refused_clearly():
    """Programs whose backward is not built (here relu attention on head dims 192 / 128, which the backward kernel does
    not cover) say so when differentiated; softmax, sigmoid and relu attention with dim_qk 128 or 64 have one
    (tests/test_bwd_gpu.py)."""
    B, H, S, D, Dv = 1, 1, 128, 192, 128
    q, k, v = [t.cuda().requires_grad_(True) for t in inputs.attention_bshd(B, H, S, D, Dv, 1)]
    o = programs.relu_engine(B, H, S, D, Dv)(q, k, v)
    with pytest.raises(NotImplementedError):
        o.sum().backward()


def test_bad_arguments_return_error_codes():
    from core.native import lib
    q, k, v = cuda(*inputs.attention_bshd(1, 1, 128, 64, 64, 1))
    o = torch.empty_like(q)
    a = lib.fill_parallel_args(q, k, v, o, mask_kind=5, fparams=[0.125])
    with pytest.raises(lib.NativeError, match="invalid argument"):
        lib.parallel_fwd(a)
    q96 = torch.zeros(1, 128, 1, 96, dtype=torch.bfloat16, device="cuda")
    a = lib.fill_parallel_args(q96, q96, q96, torch.empty_like(q96), mask_kind=0, fparams=[0.1])
    with pytest.raises(lib.NativeError, match="unsupported"):
        lib.parallel_fwd(a)
    a = lib.fill_parallel_args(q[..., 1:33], k[..., 1:33], v[..., 1:33], o[..., 1:33], mask_kind=0, fparams=[0.1])
    with pytest.raises(lib.NativeError):
        lib.parallel_fwd(a)   # misaligned base pointers are rejected before launch


@pytest.mark.parametrize("B,H,Sq,Skv,D", [(2, 8, 1, 1000, 128), (1, 4, 5, 4096, 128), (3, 2, 130, 333, 64)])
def test_mha_decode_pattern(B, H, Sq, Skv, D):
    """q_len != kv_len, equal head counts (examples/mha_decode.py): full attention of every query row over
    the whole KV, on the forward kernel."""
    g = torch.Generator().manual_seed(900 + Skv)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, H, D, generator=g).to(torch.bfloat16)
    e = programs.softmax_decode_engine(B, H, Sq, Skv, D, D)
    assert e.pattern == "mha_decode"
    o = e(q.cuda(), k.cuda(), v.cuda())
    assert o.shape == (B, Sq, H, D)
    check(o, rm.softmax_attention(q, k, v, causal=False, softmax_scale=D ** -0.5))


@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,D,is_causal", [
    (1, 8, 2, 512, 512, 128, True),      # GQA prefill, causal
    (2, 6, 3, 300, 300, 64, False),      # ragged, non-causal
    (2, 16, 4, 1, 2048, 128, False),     # dense GQA decode
])
def test_grouped_kv_heads(B, H, Hkv, Sq, Skv, D, is_causal):
    """query head h reads KV head h // (H / Hkv) (the reference's GQA templates, attn_gqa_tl.py)"""
    g = torch.Generator().manual_seed(1300 + Skv + H)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    e = programs.gqa_engine(B, H, Hkv, Sq, Skv, D, D, is_causal=is_causal)
    assert e.pattern == ("gqa" if Sq == Skv else "gqa_decode")
    o = e(q.cuda(), k.cuda(), v.cuda())
    rep = H // Hkv
    want = rm.softmax_attention(q, k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2), causal=is_causal,
                                softmax_scale=D ** -0.5)
    check(o, want)


@pytest.mark.parametrize("name,S,D", [("sliding128", 700, 128), ("two_sided", 1000, 64), ("right_open", 400, 128), ("wide_window", 2048, 128)])
def test_band_masks(name, S, D):
    """sliding-window and other band masks: KV tiles outside the band are skipped, tiles crossing an edge
    are masked element by element"""
    masks = {
        "sliding128": programs.sliding_window_mask,
        "two_sided": lambda b, h, q, kv: (kv - q <= 40) & (q - kv <= 300),
        "right_open": lambda b, h, q, kv: q - kv <= 17,
        "wide_window": lambda b, h, q, kv: (q >= kv) & (q - kv < 1000),
    }
    B, H = 2, 3
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 1500 + S)
    e = programs.masked_softmax_engine(B, H, S, D, D, masks[name])
    assert e.mask_kind == native_lib.MASK_BAND
    o = e(q.cuda(), k.cuda(), v.cuda())
    qi, ki = torch.arange(S).view(-1, 1), torch.arange(S).view(1, -1)
    keep = masks[name](0, 0, qi, ki)
    check(o, rm.softmax_attention(q, k, v, softmax_scale=D ** -0.5, keep=keep))
    lse = e.last_final_rowscales["lse"].cpu()
    s = torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * D ** -0.5
    want_lse = torch.logsumexp(s.masked_fill(~keep, float("-inf")), dim=-1)
    assert (lse - want_lse).abs().max().item() <= 2e-3


@pytest.mark.parametrize("B,H,Hkv,Sq,Skv,D,splits,causal", [
    (1, 8, 8, 1, 8192, 128, None, False),     # decode, split count planned from the SM count
    (2, 4, 2, 3, 3000, 64, 5, False),         # grouped heads, forced split count, ragged KV
    (1, 2, 2, 1024, 1024, 128, 3, True),      # split invariance under a causal mask (empty splits for early rows)
    (1, 3, 3, 200, 700, 128, 2, False),
])
def test_split_kv(B, H, Hkv, Sq, Skv, D, splits, causal):
    """KV range divided among several CTAs per (tile pair, head, batch) and combined through the log-sum-exp
    (the reference's split-KV decode kernels with OnlineFunc.combine, lower_decode.py:287-302,375-449)"""
    g = torch.Generator().manual_seed(1700 + Skv + H)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    e = programs.gqa_engine(B, H, Hkv, Sq, Skv, D, D, is_causal=causal)
    e.kv_splits = splits
    o = e(q.cuda(), k.cuda(), v.cuda())
    keep = (torch.arange(Skv).view(1, -1) <= torch.arange(Sq).view(-1, 1)) if causal else torch.ones(Sq, Skv, dtype=torch.bool)
    check(o, rm.softmax_attention(q, k, v, softmax_scale=D ** -0.5, keep=keep))
    s = torch.einsum("bshgd,bthd->bhgst", q.float().view(B, Sq, Hkv, H // Hkv, D), k.float()).reshape(B, H, Sq, Skv) * D ** -0.5
    want_lse = torch.logsumexp(s.masked_fill(~keep, float("-inf")), dim=-1)
    assert (e.last_final_rowscales["lse"].cpu() - want_lse).abs().max().item() <= 2e-3
    if splits is None:
        from attn_engine.attn_engine import plan_kv_splits
        assert plan_kv_splits(B, H, Sq, Skv, torch.device("cuda")) > 1


@pytest.mark.parametrize("B,H,S,D,Dv", [(1, 2, 384, 256, 512), (1, 3, 200, 256, 128)])
def test_wide_heads_retention_parallel(B, H, S, D, Dv):
    """dims of examples/retention_parallel.py's own run (256 / 512): one query tile per CTA, one launch per
    128-column slice of v and o"""
    g = torch.Generator().manual_seed(77 + S)
    q = (torch.randn(B, S, H, D, generator=g) * D ** -0.25).to(torch.bfloat16)
    k = (torch.randn(B, S, H, D, generator=g) * D ** -0.25).to(torch.bfloat16)
    v = torch.randn(B, S, H, Dv, generator=g).to(torch.bfloat16)
    mask = torch.rand(1, H, S, S, generator=g).tril().to(torch.bfloat16)
    e = programs.retention_parallel_engine(B, H, S, D, Dv)
    o = e(*cuda(q, k, v, mask))
    assert o.shape == (B, S, H, Dv)
    check(o, rm.retention_parallel(q, k, v, mask))


def test_wide_heads_softmax():
    B, H, S, D, Dv = 2, 2, 300, 256, 256
    g = torch.Generator().manual_seed(79)
    q = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, Dv, generator=g).to(torch.bfloat16)
    e = programs.softmax_engine(B, H, S, D, Dv, is_causal=True)
    o = e(*cuda(q, k, v))
    check(o, rm.softmax_attention(q, k, v, causal=True, softmax_scale=D ** -0.5))


def test_block_sparse_varlen_gqa_decode():
    """examples/sparse_gqa_decode.py: one query token, per-KV-head block mask (32-token blocks) and per-sequence
    cache lengths given at call time"""
    B, H, Hkv, Skv, D, block = 3, 16, 4, 1000, 128, 32
    g = torch.Generator().manual_seed(2100)
    q = torch.randn(B, 1, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, Hkv, D, generator=g).to(torch.bfloat16)
    lens = torch.tensor([1000, 517, 64], dtype=torch.int32)
    nblk = (Skv + block - 1) // block
    block_mask = torch.rand(B, Hkv, nblk, generator=g) < 0.3
    block_mask[:, :, 0] = True                       # every row keeps something
    e = programs.sparse_decode_engine(B, H, Hkv, Skv, D, D, block=block)
    o = e(q.cuda(), k.cuda(), v.cuda(), block_mask=block_mask.cuda(), cache_seqlens=lens.cuda())
    assert o.shape == (B, 1, H, D)
    keep = block_mask.repeat_interleave(block, dim=-1)[..., :Skv] & (torch.arange(Skv).view(1, 1, -1) < lens.view(-1, 1, 1))
    rep = H // Hkv
    want = torch.empty(B, 1, H, D)
    for b in range(B):
        for h in range(H):
            kk = keep[b, h // rep].view(1, Skv)
            want[b, :, h] = rm.softmax_attention(q[b:b + 1, :, h:h + 1], k[b:b + 1, :, h // rep:h // rep + 1],
                                                 v[b:b + 1, :, h // rep:h // rep + 1], softmax_scale=D ** -0.5, keep=kk)[0, :, 0]
    check(o, want)


@pytest.mark.parametrize("chunk", [1, 2, 5])
def test_forward_host_streams_batch_slices(chunk):
    """The host-buffer call (batch slices on three streams) returns what the device call returns, bit for bit."""
    B, H, S, D = 5, 3, 384, 128
    torch.manual_seed(11)
    hq, hk, hv = (torch.randn(B, S, H, D).to(torch.bfloat16).pin_memory() for _ in range(3))
    eng = programs.softmax_engine(B, H, S, D, D, is_causal=True)
    want = eng(hq.cuda(), hk.cuda(), hv.cuda())
    want_lse = eng.last_final_rowscales["lse"].clone()
    got = eng.forward_host(hq, hk, hv, batch_chunk=chunk)
    torch.cuda.synchronize()
    assert not got.is_cuda and got.is_pinned()
    assert torch.equal(got, want.cpu())
    assert torch.equal(eng.last_final_rowscales["lse"], want_lse.cpu())
    with pytest.raises(ValueError):
        eng.forward_host(hq.cuda(), hk, hv)


def test_lowered_functor_op_vocabulary():
    """Min, Abs, Neg, index operands, Exp2, Log2 and a division by a per-row value, all through the LOWERED functor
    (nothing here is recognised as a built-in): against the torch interpreter of the same traced DAG and against
    the closed form softmax(min(scale q.k, cap) - slope_h |i - j|) v."""
    from core.lower.trace import run_traced_attention
    B, H, S, D, cap, slope = 1, 3, 320, 64, 2.0, 0.02
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 12)
    e = programs.capped_distance_bias_engine(B, H, S, D, D, cap=cap, slope=slope)
    assert e.functor_kind == "lowered"
    for needle in ("fminf(", "fabsf(", "fast_exp2(", "fast_log2("):
        assert needle in e.functor_source
    o = e(*cuda(q, k, v))
    lse = e.last_final_rowscales["lse"].cpu()
    pos = torch.arange(S)
    dist = (pos.view(-1, 1) - pos.view(1, -1)).abs().float()
    s = torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * D ** -0.5
    s = s.clamp(max=cap) - dist * (slope * (torch.arange(H).float() + 1)).view(1, H, 1, 1)
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool).tril(), float("-inf"))
    want = torch.einsum("bhst,bthd->bshd", torch.softmax(s, -1), v.float())
    check(o, want)
    assert (lse - torch.logsumexp(s, -1)).abs().max().item() < 2e-3
    o_ref, fin = run_traced_attention(e.traced, q, k, v, causal=True)
    check(o, o_ref)
    assert (lse - fin["lse"]).abs().max().item() < 2e-3


def test_mha_decode_against_reference_golden():
    """golden from the reference's decode closure (testing/test.py:131-148), its tolerance 1e-2"""
    g = torch.load(os.path.join(GOLD, "mha_decode.pt"))
    B, H, Sq, KV, D, Dv = g["shape"]
    gen = torch.Generator().manual_seed(g["seed"])
    q = torch.randn(B, Sq, H, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, KV, H, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, KV, H, Dv, generator=gen).to(torch.bfloat16)
    e = programs.softmax_decode_engine(B, H, Sq, KV, D, Dv)
    for splits in (1, 2):
        e.kv_splits = splits
        o = e(*cuda(q, k, v))
        assert o.shape == (B, Sq, H, Dv)
        check(o, g["o"], max_abs=1e-2)


def test_sparse_gqa_decode_against_reference_golden():
    """golden from the reference's block-sparse decode closure (testing/test.py:654-694): 32-token blocks per
    (batch, KV head), ragged cache lengths"""
    g = torch.load(os.path.join(GOLD, "sparse_gqa_decode.pt"))
    B, H, G, S, D, Dv = g["shape"]
    gen = torch.Generator().manual_seed(g["seed"])
    q = torch.randn(B, 1, H, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, S, G, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, S, G, Dv, generator=gen).to(torch.bfloat16)
    e = programs.sparse_decode_engine(B, H, G, S, D, Dv, block=g["block"])
    o = e(*cuda(q, k, v), block_mask=g["block_mask"].cuda(), cache_seqlens=g["cache_seqlens"].cuda())
    check(o[:, 0], g["o"], max_abs=1e-2)
    check(o[:, 0], rm.sparse_gqa_decode(q, k, v, g["block_mask"], g["cache_seqlens"], g["block"]))


def test_reference_examples_called_on_the_gpu():
    """The reference's own example programs, imported unchanged from a checkout of the reference (skipped where none
    is present), constructed AND called on seeded inputs, against the oracle."""
    import importlib
    import sys
    from conftest import reference_root
    ref = reference_root()
    if ref is None:
        pytest.skip("no checkout of the reference on this machine")
    sys.path.insert(0, ref)
    try:
        B, H, S, D = 1, 4, 512, 128
        q, k, v = inputs.attention_bshd(B, H, S, D, D, 301)
        for mod_name in ("examples.mha", "examples.mha_v2"):
            eng = importlib.import_module(mod_name).causal_softmax_attention(B, H, S, D, D, dtype=torch.bfloat16)
            check(eng(*cuda(q, k, v)), rm.softmax_attention(q, k, v, True))
        bias = torch.tensor([-math.log(S)])
        for mod_name in ("examples.sigmoid_attn", "examples.sigmoid_attn_v2"):
            eng = importlib.import_module(mod_name).sigmoid_attention(B, H, S, D, D)   # fp16 engines
            qs, ks, vs = [(t * D ** -0.5 if i == 0 else t).to(eng.dtype) for i, t in enumerate((q, k, v))]
            o = eng(*cuda(qs, ks, vs), bias.cuda())
            check(o, rm.sigmoid_attention(qs, ks, vs, bias, True), max_abs=1e-1, mean_abs=1e-2)
        q6, k6, v6 = inputs.attention_bshd(1, 6, 512, 64, 64, 302, k_scale=0.5, v_scale=0.5)
        for mod_name in ("examples.reluattn", "examples.reluattn_v2"):
            eng = importlib.import_module(mod_name).relu_attention(1, 6, 512, 64, 64, dtype=torch.bfloat16)
            check(eng(*cuda(q6, k6, v6)), rm.relu_attention(q6, k6, v6), max_abs=1e-1, mean_abs=1e-2)
        dec = importlib.import_module("examples.mha_decode").softmax_attention_decode(2, 8, 1, 4096, 128, 128, dtype=torch.bfloat16)
        qd, kd, vd = inputs.randn((2, 1, 8, 128), 303, torch.bfloat16), inputs.randn((2, 4096, 8, 128), 304, torch.bfloat16), \
            inputs.randn((2, 4096, 8, 128), 305, torch.bfloat16)
        check(dec(*cuda(qd, kd, vd)), rm.softmax_attention(qd, kd, vd, causal=False))
        ret = importlib.import_module("examples.retnet_recurrent").retnet_recurrent(1, 8, 512, 256, 512, dtype=torch.bfloat16)
        qr, kr, vr, decay = inputs.retention_bhsd(1, 8, 512, 256, 512, 306)
        torch.testing.assert_close(ret(*cuda(qr, kr, vr, decay)).float().cpu(), rm.retention_recurrent(qr, kr, vr), rtol=1e-1, atol=1e-1)
        gla = importlib.import_module("examples.gated_retention").gated_retention(1, 4, 512, 256, 256, dtype=torch.bfloat16)
        qg, kg, vg, gg = inputs.gla_inputs(1, 4, 512, 256, 256, 307)
        torch.testing.assert_close(gla(*cuda(qg, kg, vg, gg)).float().cpu(),
                                   rm.decayed_linear_attention(qg, kg, vg, gg, scale=256 ** -0.5), rtol=1e-1, atol=1e-1)
    finally:
        sys.path.remove(ref)


def _masked_oracle(q, k, v, mask_mod, per_head):
    """softmax attention under an arbitrary mask_mod, head by head when the mask depends on (batch, head)"""
    B, S, H, _ = q.shape
    Skv = k.shape[1]
    qi, ki = torch.arange(S).view(-1, 1), torch.arange(Skv).view(1, -1)
    if not per_head:
        return rm.softmax_attention(q, k, v, keep=mask_mod(0, 0, qi, ki).expand(S, Skv))
    out = torch.empty(B, S, H, v.shape[-1])
    for b in range(B):
        for h in range(H):
            keep = mask_mod(torch.tensor(b), torch.tensor(h), qi, ki).expand(S, Skv)
            out[b, :, h] = rm.softmax_attention(q[b:b + 1, :, h:h + 1], k[b:b + 1, :, h:h + 1], v[b:b + 1, :, h:h + 1], keep=keep)[0, :, 0]
    return out


GENERAL_MASKS = {
    # causal inside documents of 192 tokens: partial tiles on and next to the diagonal, everything else skipped
    "document": (lambda b, h, q, kv: (q // 192 == kv // 192) & (q >= kv), False),
    # whole KV tiles dropped in a checkerboard, the diagonal kept: full tiles and skipped tiles only
    "checkerboard": (lambda b, h, q, kv: (((q // 128) + (kv // 128)) % 2 == 0) | (q == kv), False),
    # a different causal offset for every head, first column always kept
    "per_head_offset": (lambda b, h, q, kv: (q >= kv + 64 * h) | (kv == 0), True),
    # a prefix whose length depends on the batch entry, causal behind it
    "per_batch_prefix": (lambda b, h, q, kv: (kv <= q) | (kv < 100 * (b + 1)), True),
}


@pytest.mark.parametrize("name", sorted(GENERAL_MASKS))
@pytest.mark.parametrize("S,D", [(600, 64), (1024, 128)])
def test_general_masks_run_as_block_sparse_walks(name, S, D):
    """mask_mod that is neither causal nor a band, or that uses the batch / head index: the reference switches to its
    block-sparse template (core/lower/lower.py:723-738); here the KV tiles without a kept position are skipped and the
    partially kept ones carry their element mask."""
    mask_mod, per_head = GENERAL_MASKS[name]
    B, H = 2, 3
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 500 + S)
    e = programs.masked_softmax_engine(B, H, S, D, D, mask_mod)
    assert e.sparse_walk and e.functor_kind == "builtin_softmax"
    assert (e._sparse_host["batch"], e._sparse_host["heads"]) == ((B, H) if per_head else (1, 1))
    o = e(*cuda(q, k, v))
    check(o, _masked_oracle(q, k, v, mask_mod, per_head))


def test_general_mask_with_a_lowered_functor_and_empty_query_tiles():
    """sigmoid attention (lowered, identity online function) under a mask that leaves the second query tile of the first
    batch entry without any KV tile: those rows are the epilogue of an empty accumulator, i.e. zero"""
    B, H, S, D = 2, 2, 512, 64
    mask_mod = lambda b, h, q, kv: (kv <= q) & ((q < 128) | (q >= 256) | (b > 0))   # noqa: E731
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 77)
    bias = torch.tensor([-math.log(S)])
    score_mod = lambda s, c, b, h, qi, ki: ((s * D ** -0.5 + c.input_tensors["softmax_bias"]) * 0.5).tanh() * 0.5 + 0.5   # noqa: E731
    from attn_engine import AttentionEngine
    from core import CustomIO
    e = AttentionEngine(programs._meta(B, H, S, D, D, torch.bfloat16), CustomIO({"softmax_bias": (1,)}), score_mod=score_mod,
                        mask_mod=mask_mod, online_func=None)
    assert e.sparse_walk and e.functor_kind == "lowered"
    o = e(*cuda(q, k, v), bias.cuda())
    qi, ki = torch.arange(S).view(-1, 1), torch.arange(S).view(1, -1)
    want = torch.empty(B, S, H, D)
    for b in range(B):
        s = torch.einsum("shd,thd->hst", q[b].float(), k[b].float()) * D ** -0.5 + bias
        p = torch.sigmoid(s) * mask_mod(torch.tensor(b), 0, qi, ki)
        want[b] = torch.einsum("hst,thd->shd", p, v[b].float())
    check(o, want)
    assert bool((o[0, 128:256] == 0).all())


@pytest.mark.parametrize("online", ["softmax", "abssum"])
def test_split_kv_with_a_lowered_combine(online):
    """Split-KV for a LOWERED functor: the user's OnlineFunc.combine (traced over the splits' final row scales, lowered
    with column reductions) weighs the partial results; forced split counts against the unsplit run and the closed form."""
    from core.lower.trace import run_traced_combine
    B, H, Sq, Skv, D = 2, 3, 2, 1152, 128     # 9 KV tiles
    g = torch.Generator().manual_seed(2200)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, Skv, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Skv, H, D, generator=g).to(torch.bfloat16)
    e = programs.split_decode_engine(B, H, Sq, Skv, D, D, online=online)
    assert e.functor_kind == "lowered" and e.traced.combine_out is not None
    assert "for (int k = 0; k < n; ++k)" in e.functor_source
    if online == "softmax":
        want = rm.softmax_attention(q, k, v, causal=False)
    else:
        s = torch.einsum("bshd,bthd->bhst", q.float(), k.float()) * D ** -0.5
        want = torch.einsum("bhst,bthd->bshd", s / s.abs().sum(-1, keepdim=True).clamp(min=1.0), v.float())
    outs = {}
    for splits in (1, 2, 3, 4, 9):      # 4 becomes 3 (no split may be empty)
        e.kv_splits = splits
        outs[splits] = e(*cuda(q, k, v))
        check(outs[splits], want)
    assert torch.equal(outs[4], outs[3])
    # the lowered combine means what the traced one means
    lse = torch.tensor([[1.0, 2.0], [0.5, -1.0], [3.0, 0.0]])
    fin = {name: (lse if name in ("lse", "den") else lse.abs() + 1) for name in e.traced.final}
    w = run_traced_combine(e.traced, fin)
    assert w.shape == (3, 2) and torch.isfinite(w).all()
    if online == "softmax":
        assert torch.allclose(w, torch.softmax(lse, 0), atol=1e-6)


@pytest.mark.parametrize("B,H,S,D,Dv", [(1, 16, 2048, 128, 256), (1, 16, 2048, 192, 128), (2, 3, 333, 192, 128), (1, 2, 400, 128, 384)])
def test_head_dims_of_the_reference_suite(B, H, S, D, Dv):
    """dim_qk 128 / dim_v 256 (the reference's second softmax case, testing/test.py:55) and 192 / 128 (its H100
    sweep, testing/benchmark_h100.py:60-63): causal softmax against the oracle"""
    g = torch.Generator().manual_seed(D + Dv)
    q = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, Dv, generator=g).to(torch.bfloat16)
    e = programs.softmax_engine(B, H, S, D, Dv, is_causal=True)
    o = e(*cuda(q, k, v))
    assert o.shape == (B, S, H, Dv)
    check(o, rm.softmax_attention(q, k, v, causal=True, softmax_scale=D ** -0.5))
    assert (e.last_final_rowscales["lse"].cpu() - rm.softmax_lse(q, k, True, D ** -0.5)).abs().max().item() < 1e-3


def test_decode_tiles_entry_point():
    """attn_b200_decode_tiles against a torch evaluation of the same rule, bit for bit"""
    import numpy as np
    B, Hkv, Skv, block = 3, 2, 1000, 32
    g = torch.Generator().manual_seed(5)
    nblk = (Skv + block - 1) // block
    bm = torch.rand(B, Hkv, nblk, generator=g) < 0.4
    lens = torch.tensor([1000, 517, 1], dtype=torch.int32)
    sp = native_lib.decode_tiles(bm.cuda(), lens.cuda(), B, Hkv, Skv, block, torch.device("cuda", 0))
    torch.cuda.synchronize()
    keep = bm.repeat_interleave(block, -1)[..., :Skv] & (torch.arange(Skv).view(1, 1, -1) < lens.view(-1, 1, 1))
    tiles = torch.nn.functional.pad(keep, (0, 1024 - Skv)).view(B, Hkv, 8, 128)
    col = sp["elem_mask"].cpu().numpy().view(np.uint32).reshape(B, Hkv, 8, 4)
    bits = ((col[..., None] >> np.arange(32, dtype=np.uint32)) & 1).reshape(B, Hkv, 8, 128).astype(bool)
    assert np.array_equal(bits, tiles.numpy())
    kept_words = sp["keep"].cpu().numpy().view(np.uint32).reshape(B, Hkv)
    part_words = sp["partial"].cpu().numpy().view(np.uint32).reshape(B, Hkv)
    any_, all_ = tiles.any(-1).numpy(), tiles.all(-1).numpy()
    for b in range(B):
        for h in range(Hkv):
            assert [(int(kept_words[b, h]) >> j) & 1 for j in range(8)] == [int(x) for x in any_[b, h]]
            assert [(int(part_words[b, h]) >> j) & 1 for j in range(8)] == [int(x and not y) for x, y in zip(any_[b, h], all_[b, h])]
