"""The block-mask helpers of the front-end (core/transform/core.py) against the committed outputs of the reference's
own helpers (attention_engine/core/transform/core.py:455-506: create_block_mask, create_block_idx, is_causal_mask,
is_less_causal_mask), produced by tests/golden/make_golden.py.  Integer work: compared bit for bit."""

import importlib.util
import os

import pytest
import torch

from core.transform.core import create_block_idx, create_block_mask, is_causal_mask, is_less_causal_mask

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)
GOLD = torch.load(os.path.join(HERE, "golden", "block_masks.pt"))


@pytest.mark.parametrize("mask_name", sorted(make_golden.MASK_CASES))
def test_block_masks_bit_exact(mask_name):
    fn = make_golden.MASK_CASES[mask_name]
    for shape in make_golden.MASK_SHAPES:
        want = GOLD[(mask_name, shape)]
        B, H, Q, KV, bq, bk = shape
        bm = create_block_mask(fn, B, H, Q, KV, "cpu", bq, bk)
        assert bm.dtype == torch.int8 and torch.equal(bm, want["block_mask"]), (mask_name, shape)
        assert bool(is_causal_mask(bm, bq, bk)) == want["is_causal"]
        assert bool(is_less_causal_mask(bm, bq, bk)) == want["is_less_causal"]
        assert torch.equal(create_block_idx(fn, B, H, Q, KV, "cpu", bq, bk), want["block_idx"])
