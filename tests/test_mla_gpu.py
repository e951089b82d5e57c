"""Parity of the sm_100a MLA decode kernels (split-KV + combine, through the engine API and the C ABI)
against the CPU oracle and the committed golden output of the reference's PyTorch closure.
Tolerance: max-abs <= 2e-2, mean-abs <= 2e-3 for the 16-bit output against the fp32 reference."""

import os

import pytest
import torch

from examples_b200 import programs
from attn_engine.mla import flash_mla_with_kvcache, mla_decode_forward, plan_splits
from core.native import lib
from oracle import inputs, reference_math as rm

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def check(o, want, max_abs=2e-2, mean_abs=2e-3):
    assert lib.last_device_status() == 0
    o = o.float().cpu().reshape(want.shape)
    assert torch.isfinite(o).all()
    d = (o - want.float()).abs()
    assert d.max().item() <= max_abs and d.mean().item() <= mean_abs, (d.max().item(), d.mean().item())


def oracle(q, kv, Dv):
    return rm.mla_decode(q[..., :Dv], q[..., Dv:], kv[..., :Dv], kv[..., Dv:])


def test_against_reference_golden_tl_convention():
    g = torch.load(os.path.join(GOLD, "mla.pt"))
    B, H, S, D, Dv = g["shape"]
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, g["seed"])
    e = programs.mla_engine(B, H, S, D, Dv)
    qc, kvc = q.cuda(), kv.cuda()
    # separate nope / rope tensors, as the reference's TileLang path is called
    o = e(qc[..., :Dv].contiguous(), qc[..., Dv:].contiguous(), kvc[..., :Dv].contiguous(), kvc[..., Dv:].contiguous())
    assert o.shape == (B, 1, H, Dv)
    check(o, g["o"])


@pytest.mark.parametrize("B,H,S,splits", [
    (2, 128, 1024, 1), (2, 128, 1024, 4), (1, 128, 8192, None), (3, 64, 500, 3), (1, 16, 37, 1),
    (1, 128, 297, 2), (2, 256, 640, 2), (1, 128, 129, 1),
])
def test_shapes_and_splits(B, H, S, splits):
    D, Dv = 576, 512
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 1000 + S)
    o, lse = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5, num_splits=splits)
    check(o, oracle(q, kv, Dv))
    want_lse = rm.mla_decode_lse(q[..., :Dv], q[..., Dv:], kv[..., :Dv], kv[..., Dv:])
    assert (lse.cpu() - want_lse).abs().max().item() < 2e-3


def test_split_invariance_property():
    """Size-independent property: the result does not depend on how the KV range is split."""
    B, H, S, D, Dv = 2, 128, 4096, 576, 512
    q, kv = [t.cuda() for t in inputs.mla_inputs(B, H, S, D, Dv, 77)]
    outs = [mla_decode_forward(q, kv, Dv, D ** -0.5, num_splits=s)[0].float() for s in (1, 2, 5, 16)]
    for o in outs[1:]:
        assert (o - outs[0]).abs().max().item() < 8e-3


def test_paged_convention_returns_out_and_lse():
    B, H, S, D, Dv = 2, 128, 2048, 576, 512
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 5)
    e = programs.mla_engine(B, H, S, D, Dv, backend="cute")
    pages = kv.cuda().view(B * S // 64, 64, 1, D)
    out, lse = e(q.cuda(), pages)
    assert out.shape == (B, 1, H, Dv) and lse.shape == (B, H, 1)
    check(out, oracle(q, kv, Dv))


def test_fp16():
    B, H, S, D, Dv = 1, 128, 768, 576, 512
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 6, dtype=torch.float16)
    o, _ = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5, num_splits=2)
    check(o, oracle(q, kv, Dv))


def test_config5_full_size_sampled_sequences():
    """BASELINE config 5 (B=128, 128 heads, 8192 tokens, 576/512) at full size; oracle on sampled sequences."""
    c = inputs.CONFIGS["C5"]
    B, H, S, D, Dv = c["B"], c["H"], c["S"], c["D"], c["Dv"]
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, c["seed"])
    o, lse = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5)
    assert lib.last_device_status() == 0
    o = o.cpu()
    assert torch.isfinite(o.float()).all()
    for b in (0, 63, 127):
        check(o[b:b + 1], oracle(q[b:b + 1], kv[b:b + 1], Dv))


def test_plan_and_workspace_errors():
    # 128 sequences on 74 clusters leave the second round far from full: scheduled (0); 148 fill two rounds: one split
    assert plan_splits(128, 128, 8192, 576, 512, 148) == 0
    assert plan_splits(148, 128, 8192, 576, 512, 148) == 1
    assert plan_splits(2, 128, 8192, 576, 512, 148) >= 0
    q, kv = [t.cuda() for t in inputs.mla_inputs(1, 128, 256, 576, 512, 1)]
    tiny = torch.empty(16, dtype=torch.uint8, device="cuda")
    o, _ = mla_decode_forward(q, kv, 512, 576 ** -0.5, num_splits=2, workspace=tiny)   # too small: replaced internally
    check(o, oracle(q.cpu(), kv.cpu(), 512))
    import ctypes as C
    a = lib.MlaArgs()
    a.q, a.kv, a.o = q.data_ptr(), kv.data_ptr(), o.data_ptr()
    a.q_stride[:] = (128 * 576, 576)
    a.kv_stride[:] = (256 * 576, 576)
    a.shape = lib.MlaShape(1, 128, 256, 576, 512)
    a.num_splits, a.dtype, a.scale = 2, 1, 0.04
    assert lib.load_library().attn_b200_mla_decode(C.byref(a), None) == -5      # no workspace
    a.shape = lib.MlaShape(1, 128, 256, 512, 512)
    assert lib.load_library().attn_b200_mla_decode(C.byref(a), None) == -2      # unsupported dims


def ragged_oracle(q, kv, lens, Dv):
    """per sequence: attention over its first lens[b] cache rows"""
    outs, lses = [], []
    for b, n in enumerate(lens):
        qb, kb = q[b:b + 1], kv[b:b + 1, :n]
        outs.append(rm.mla_decode(qb[..., :Dv], qb[..., Dv:], kb[..., :Dv], kb[..., Dv:]))
        lses.append(rm.mla_decode_lse(qb[..., :Dv], qb[..., Dv:], kb[..., :Dv], kb[..., Dv:]))
    return torch.cat(outs), torch.cat(lses)


@pytest.mark.parametrize("splits", [1, 3])
def test_ragged_sequence_lengths(splits):
    """cache_seqlens of flash_api.cpp:61-72: every sequence stops at its own length; the rows behind it
    hold large numbers that must not leak into the result."""
    B, H, S, D, Dv = 5, 128, 700, 576, 512
    lens = [700, 1, 129, 64, 333]
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 4001)
    kv_dirty = kv.clone()
    for b, n in enumerate(lens):
        kv_dirty[b, n:] = 1000.0
    o, lse = mla_decode_forward(q.cuda(), kv_dirty.cuda(), Dv, D ** -0.5, num_splits=splits,
                                cache_seqlens=torch.tensor(lens, dtype=torch.int32, device="cuda"))
    want, want_lse = ragged_oracle(q, kv, lens, Dv)
    check(o, want)
    assert (lse.cpu().reshape(-1) - want_lse.reshape(-1)).abs().max().item() <= 2e-3


@pytest.mark.parametrize("page,splits", [(64, 1), (64, 4), (128, 2)])
def test_paged_cache_with_block_table(page, splits):
    """block_table of flash_api.cpp:61-72 / flash_mla_interface.py:74-115: the cache is a pool of pages in
    arbitrary order, with unrelated pages (large numbers) in between."""
    B, H, S, D, Dv = 3, 128, 1024, 576, 512
    lens = [1024, 450, 65]
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 4002)
    blocks = S // page
    gen = torch.Generator().manual_seed(7)
    num_pages = B * blocks + 5
    perm = torch.randperm(num_pages, generator=gen)[: B * blocks].view(B, blocks)
    pool = torch.full((num_pages, page, 1, D), 1000.0, dtype=kv.dtype)
    for b in range(B):
        for i in range(blocks):
            pool[perm[b, i], :, 0] = kv[b, i * page:(i + 1) * page, 0]
    table = perm.to(torch.int32)
    # entries behind a sequence's last page are never read: make them invalid
    for b, n in enumerate(lens):
        table[b, (n + page - 1) // page:] = -1
    out, lse = flash_mla_with_kvcache(q.cuda(), pool.cuda(), table.cuda(),
                                      torch.tensor(lens, dtype=torch.int32, device="cuda"), Dv, None, splits)
    assert out.shape == (B, 1, H, Dv) and lse.shape == (B, H, 1)
    want, want_lse = ragged_oracle(q, kv, lens, Dv)
    check(out, want)
    assert (lse.cpu().reshape(-1) - want_lse.reshape(-1)).abs().max().item() <= 2e-3


def reference_schedule(seqlens, block, overhead, parts):
    """The equal-payload partition of the reference's scheduler (kernels/get_mla_metadata.cu:22-71) restated on
    Python ints with its block size and fixed overhead as parameters: returns (records [parts][5] = begin sequence,
    begin token, end sequence, end token, begin split index; cumulative split counts [batch + 1])."""
    batch = len(seqlens)
    blocks = [-(-n // block) for n in seqlens]
    total = sum(nb + overhead for nb in blocks)
    payload = max(-(-total // parts) + overhead, 2 * overhead)
    recs, cum = [], [0] * (batch + 1)
    idx = blk = split = acc = 0
    for _ in range(parts):
        rec = [idx, blk * block, 0, 0, split]
        remain = payload
        while idx < batch:
            rest = blocks[idx] - blk
            if remain >= rest + overhead:
                acc += split + 1
                cum[idx + 1] = acc
                remain -= rest + overhead
                idx, blk, split = idx + 1, 0, 0
            else:
                if remain - overhead > 0:
                    blk += remain - overhead
                    split += 1
                break
        rec[2] = idx if blk > 0 else idx - 1
        rec[3] = blk * block if blk > 0 else seqlens[idx - 1]
        recs.append(rec)
    assert idx == batch and blk == 0 and split == 0
    return recs, cum


@pytest.mark.parametrize("batch,max_len,seed", [(128, 8192, 1), (5, 30000, 2), (300, 700, 3), (1, 100000, 4), (74, 4096, 5)])
def test_tile_scheduler_matches_the_reference_algorithm_bit_for_bit(batch, max_len, seed):
    """attn_b200_mla_metadata (device) against the restated reference algorithm (integers: exact), and the properties
    that make it a schedule: every KV tile of every sequence is covered exactly once, in order, and no part carries
    more than the payload."""
    from attn_engine.mla import mla_schedule, num_parts
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, max_len + 1, (batch,), generator=g).to(torch.int32)
    if seed == 1:
        lens[:] = max_len      # the dense benchmark case
    dev = torch.device("cuda", 0)
    meta, cum = mla_schedule(lens.cuda(), batch, max_len, 128, dev)
    torch.cuda.synchronize()
    parts = num_parts(128, dev)
    want, want_cum = reference_schedule([int(x) for x in lens], 128, 4, parts)
    assert meta.shape == (parts, 8)
    assert meta[:, :5].cpu().tolist() == want
    assert cum.cpu().tolist() == want_cum
    # coverage
    tiles = [-(-int(n) // 128) for n in lens]
    seen = [0] * batch
    for rec in meta.cpu().tolist():
        b0, t0, b1, end_tok = rec[0], rec[1] // 128, rec[2], rec[3]
        took = 0
        for b in range(b0, min(b1, batch - 1) + 1):
            lo = t0 if b == b0 else 0
            hi = min(tiles[b], -(-end_tok // 128)) if b == b1 else tiles[b]
            assert lo == seen[b]
            seen[b] = hi
            took += hi - lo
        assert took == rec[5]
    assert seen == tiles
    total = sum(t + 4 for t in tiles)
    assert max(rec[5] for rec in meta.cpu().tolist()) <= max(-(-total // parts) + 4, 8)


@pytest.mark.parametrize("B,H,S", [(3, 128, 5000), (1, 128, 20000), (200, 128, 600), (9, 256, 3000), (2, 64, 130)])
def test_scheduled_decode_ragged_lengths(B, H, S):
    """The scheduled mode (the default): clusters walk pieces of sequences cut where the equal payload ends; ragged
    lengths, a single long sequence spread over all clusters, more sequences than clusters, two head blocks."""
    D, Dv = 576, 512
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 3000 + S)
    g = torch.Generator().manual_seed(S)
    lens = torch.randint(max(1, S // 10), S + 1, (B,), generator=g).to(torch.int32)
    lens[0] = S
    o, lse = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5, cache_seqlens=lens.cuda())
    want = torch.empty(B, 1, H, Dv)
    want_lse = torch.empty(B, H)
    for b in range(B):
        n = int(lens[b])
        want[b] = oracle(q[b:b + 1], kv[b:b + 1, :n], Dv)[0]
        want_lse[b] = rm.mla_decode_lse(q[b:b + 1, ..., :Dv], q[b:b + 1, ..., Dv:], kv[b:b + 1, :n, :, :Dv], kv[b:b + 1, :n, :, Dv:])[0]
    check(o, want)
    assert (lse.cpu() - want_lse).abs().max().item() < 2e-3
    # the same through a schedule made once and passed in, and against a uniform split: identical pieces, identical bits
    from attn_engine.mla import mla_schedule
    meta, cum = mla_schedule(lens.cuda(), B, S, H, torch.device("cuda", 0))
    o2, lse2 = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5, cache_seqlens=lens.cuda(), tile_scheduler_metadata=meta,
                                  num_splits_cum=cum)
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    o3, _ = mla_decode_forward(q.cuda(), kv.cuda(), Dv, D ** -0.5, cache_seqlens=lens.cuda(), num_splits=1)
    check(o3, want)


def test_reference_call_with_scheduler_metadata():
    """get_mla_metadata + flash_mla_with_kvcache used the way the reference's benchmark uses them
    (testing/benchmark_h100.py:1079-1087): metadata once, then the paged decode call"""
    from attn_engine.mla import get_mla_metadata
    B, H, S, D, Dv, page = 4, 128, 1024, 576, 512, 64
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 44)
    lens = torch.tensor([1024, 700, 64, 333], dtype=torch.int32)
    pages = S // page
    table = torch.arange(B * pages, dtype=torch.int32).view(B, pages)
    pool = kv.view(B * pages, page, 1, D)
    meta, nsplits = get_mla_metadata(lens.cuda(), H, 1)
    assert meta.dtype == torch.int32 and meta.shape[1] == 8 and nsplits.shape == (B + 1,)
    out, lse = flash_mla_with_kvcache(q.cuda(), pool.cuda(), table.cuda(), lens.cuda(), Dv, meta, nsplits)
    assert out.shape == (B, 1, H, Dv) and lse.shape == (B, H, 1)
    want = torch.cat([oracle(q[b:b + 1], kv[b:b + 1, :int(lens[b])], Dv) for b in range(B)])
    check(out, want)
