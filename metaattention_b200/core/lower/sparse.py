"""Block-sparse walks for the forward kernel: from a ``mask_mod`` to the per-query-tile bitmaps of KV tiles and the
element masks of partially kept tiles that ``AttnB200ParallelArgs.tile_keep`` / ``tile_partial`` / ``elem_mask``
describe (include/attn_b200.h).

The reference infers a block mask from ``mask_mod`` and switches to its block-sparse template when the mask is not
causal (attention_engine/core/lower/lower.py:723-738, core/transform/core.py:407-506), evaluating ``mask_mod``
element-wise inside kept blocks through generated code (core/template/tl_template/attn/blockattn_tl.py:168-200).
Here the mask function is evaluated once on the CPU, at construction: blocks without a kept position are never
visited, blocks kept completely need nothing, and the rest carry their 128x128 keep bits with them, so any Python
``mask_mod`` works, whether or not it could be translated to device code.
"""

from __future__ import annotations

import numpy as np
import torch

from core.transform.core import _eval_mask_2d, mask_depends_on_batch_head

TILE = 128


def _pack_bits(bits: torch.Tensor) -> torch.Tensor:
    """bool [..., 32*k] -> int32 [..., k]; bit (c & 31) of word c >> 5 = element c."""
    shape = bits.shape[:-1] + (bits.shape[-1] // 32, 32)
    weights = (1 << np.arange(32, dtype=np.uint64))
    words = (bits.reshape(shape).numpy().astype(np.uint64) * weights).sum(-1).astype(np.uint32)
    return torch.from_numpy(words.view(np.int32))


def tiles_of_mask(dense: torch.Tensor):
    """(kept [nq, nk] bool, partial [nq, nk] bool, tiles [nq, nk, 128, 128] bool view of the zero-padded mask) for a
    dense keep-mask [q_len, kv_len].  A tile is partial when it keeps some but not all of its positions inside the
    sequence bounds."""
    q_len, kv_len = dense.shape
    nq, nk = -(-q_len // TILE), -(-kv_len // TILE)
    pad = (0, nk * TILE - kv_len, 0, nq * TILE - q_len)
    lo = torch.nn.functional.pad(dense, pad, value=False).view(nq, TILE, nk, TILE).permute(0, 2, 1, 3)
    hi = torch.nn.functional.pad(dense, pad, value=True).view(nq, TILE, nk, TILE).permute(0, 2, 1, 3)
    kept = lo.any(dim=(2, 3))
    full = hi.all(dim=(2, 3))
    return kept, kept & ~full, lo


def build_block_sparse(mask_mod, B: int, H: int, q_len: int, kv_len: int) -> dict:
    """Host-side description of the sparse walk of ``mask_mod`` (CPU tensors; ``to_device`` moves them):
    keep / partial bitmaps int32 [SB, SH, nq, words], mask_base int32 [SB, SH, nq], elem_mask int32
    [n_partial, 128, 4], with SB = B and SH = H only when the mask depends on batch or head (else 1)."""
    per_bh = mask_depends_on_batch_head(mask_mod, B, H, q_len, kv_len, "cpu")
    SB, SH = (B, H) if per_bh else (1, 1)
    nq, nk = -(-q_len // TILE), -(-kv_len // TILE)
    words = -(-nk // 32)
    keep = torch.zeros(SB, SH, nq, words * 32, dtype=torch.bool)
    part = torch.zeros(SB, SH, nq, words * 32, dtype=torch.bool)
    masks = []
    for b in range(SB):
        for h in range(SH):
            kept, partial, tiles = tiles_of_mask(_eval_mask_2d(mask_mod, b, h, q_len, kv_len, "cpu"))
            keep[b, h, :, :nk] = kept
            part[b, h, :, :nk] = partial
            if bool(partial.any()):
                masks.append(_pack_bits(tiles[partial].contiguous()))   # [n, 128, 4], (query tile, KV tile) order
    counts = part.sum(-1).reshape(-1)
    base = torch.cumsum(counts, 0) - counts
    elem = torch.cat(masks) if masks else torch.zeros(1, TILE, 4, dtype=torch.int32)
    out_bits = {}
    if not per_bh:   # the backward takes the keep matrix and its transpose as bits (one matrix for all batches and heads)
        out_bits["bits_q"], out_bits["bits_kv"], out_bits["tiles_q"], out_bits["tiles_kv"] = mask_bit_matrices(
            _eval_mask_2d(mask_mod, 0, 0, q_len, kv_len, "cpu"))
    return {**out_bits, "keep": _pack_bits(keep), "partial": _pack_bits(part), "mask_base": base.to(torch.int32).view(SB, SH, nq),
            "elem_mask": elem.contiguous(), "batch": SB, "heads": SH, "mask_rows": TILE,
            "kept_tiles": int(keep.sum()), "partial_tiles": int(part.sum()), "all_tiles": SB * SH * nq * nk}


def mask_bit_matrices(dense: torch.Tensor):
    """The keep matrix [q_len, kv_len] of a mask and its transpose as the bit tensors the backward kernels take
    (include/attn_b200.h, ATTN_B200_MASK_BITS): int32 [nq*128, nk, 4] and [nk*128, nq, 4], zero-padded to whole tiles,
    and the bitmaps of the tile pairs that keep anything, int32 [nq, ceil(nk/32)] and its transpose [nk, ceil(nq/32)]."""
    q_len, kv_len = dense.shape
    nq, nk = -(-q_len // TILE), -(-kv_len // TILE)
    padded = torch.nn.functional.pad(dense, (0, nk * TILE - kv_len, 0, nq * TILE - q_len), value=False)
    bits_q = _pack_bits(padded.contiguous()).view(nq * TILE, nk, 4)
    bits_kv = _pack_bits(padded.t().contiguous()).view(nk * TILE, nq, 4)
    kept = padded.view(nq, TILE, nk, TILE).any(dim=3).any(dim=1)   # [nq, nk]
    pad_to = lambda m: torch.nn.functional.pad(m, (0, -m.shape[1] % 32), value=False)   # noqa: E731
    tiles_q = _pack_bits(pad_to(kept).contiguous())
    tiles_kv = _pack_bits(pad_to(kept.t()).contiguous())
    return bits_q.contiguous(), bits_kv.contiguous(), tiles_q.contiguous(), tiles_kv.contiguous()


def to_device(sparse: dict, device) -> dict:
    out = dict(sparse)
    for key in ("keep", "partial", "mask_base", "elem_mask", "bits_q", "bits_kv", "tiles_q", "tiles_kv"):
        if sparse.get(key) is not None:
            out[key] = sparse[key].to(device)
    return out
