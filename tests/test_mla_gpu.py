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
    assert plan_splits(128, 128, 8192, 576, 512, 148) >= 1
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
