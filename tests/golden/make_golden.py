"""Generates tests/golden/*.pt: outputs of the REFERENCE's own PyTorch reference
closures on seeded inputs.  Run in a container that has the reference checkout:

    python tests/golden/make_golden.py [/path/to/reference]

(default: $ATTN_B200_REFERENCE, then baseline/_ref/ of this repository, then the checkout the build environment provides)

The reference's functional suite (testing/test.py) cannot be imported as a
module (it needs termcolor, matplotlib and a GPU at import time), so the
closures -- plain functions nested inside the test functions -- are located
with `ast`, and their source is executed unchanged with torch/einops in
scope.  Nothing from the reference is written into this repository except
the numeric outputs.  The fixtures pin oracle/reference_math.py
(tests/test_oracle_golden.py)."""

import ast
import math
import os
import sys

import torch
import torch.nn.functional as F
from einops import einsum, rearrange, repeat

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import inputs  # noqa: E402


# mask functions whose block masks are pinned (name -> mask_mod); tests/test_oracle_golden.py imports this table
MASK_CASES = {
    "causal": lambda b, h, q, kv: q >= kv,
    "full": lambda b, h, q, kv: q >= 0,
    "sliding_window_100": lambda b, h, q, kv: (q >= kv) & (q - kv < 100),
    "band_70_40": lambda b, h, q, kv: (kv - q <= 40) & (q - kv <= 70),
    "per_head_offset": lambda b, h, q, kv: q >= kv + 64 * h,
    "per_batch_prefix": lambda b, h, q, kv: (kv <= q) | (kv < 32 * (b + 1)),
    "checker": lambda b, h, q, kv: ((q // 64) + (kv // 64)) % 2 == 0,
    "document": lambda b, h, q, kv: (q // 192 == kv // 192) & (q >= kv),
}
# (batch, heads, q_len, kv_len, q block, kv block)
MASK_SHAPES = [(2, 3, 512, 512, 128, 128), (1, 2, 384, 384, 64, 64), (2, 2, 256, 256, 128, 64)]


def block_mask_goldens(ref_root):
    """int8 block masks, index lists and the two causal predicates from the reference's own helpers
    (attention_engine/core/transform/core.py:455-506), imported from its checkout."""
    sys.path.insert(0, os.path.join(ref_root, "attention_engine"))
    for name in [m for m in sys.modules if m == "core" or m.startswith("core.")]:
        del sys.modules[name]   # our own top-level ``core`` package may be loaded already
    import importlib
    ref = importlib.import_module("core.transform.core")
    out = {}
    for mname, fn in MASK_CASES.items():
        for shape in MASK_SHAPES:
            B, H, Q, KV, bq, bk = shape
            bm = ref.create_block_mask(fn, B, H, Q, KV, "cpu", bq, bk)
            out[(mname, shape)] = dict(block_mask=bm.clone(), is_causal=bool(ref.is_causal_mask(bm, bq, bk)),
                                       is_less_causal=bool(ref.is_less_causal_mask(bm, bq, bk)),
                                       block_idx=ref.create_block_idx(fn, B, H, Q, KV, "cpu", bq, bk).clone())
    sys.path.pop(0)
    for name in [m for m in sys.modules if m == "core" or m.startswith("core.")]:
        del sys.modules[name]
    return out


def extract(tree, source, outer: str, inner: str, extra_globals=None, edit=None):
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == outer:
            for sub in ast.walk(node):
                if isinstance(sub, ast.FunctionDef) and sub.name == inner and sub is not node:
                    seg = ast.get_source_segment(source, sub)
                    import textwrap
                    ns = {"torch": torch, "F": F, "rearrange": rearrange, "einsum": einsum, "repeat": repeat,
                          "math": math}
                    ns.update(extra_globals or {})
                    if edit is not None:
                        seg = edit(seg)
                    exec(textwrap.dedent(seg), ns)
                    return ns[inner]
    raise KeyError(f"{outer}.{inner} not found")


def main():
    sys.path.insert(0, os.path.dirname(HERE))
    from conftest import reference_root
    ref_root = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    if ref_root is None:
        raise SystemExit("no checkout of the reference found: pass its path")
    path = os.path.join(ref_root, "testing", "test.py")
    source = open(path).read()
    tree = ast.parse(source)
    torch.set_grad_enabled(False)
    out = {}

    # softmax MHA (testing/test.py:79-104), causal and non-causal, fp32 and bf16-rounded inputs
    ref = extract(tree, source, "test_softmaxattention", "ref")
    for name, (B, H, S, D, causal, seed, dt) in {
        "softmax_c1": (1, 4, 512, 64, False, 1001, torch.float32),          # BASELINE config 1, full size
        "softmax_causal_small": (2, 3, 192, 128, True, 11, torch.bfloat16),
        "softmax_noncausal_d64": (1, 2, 160, 64, False, 12, torch.bfloat16),
    }.items():
        q, k, v = inputs.attention_bshd(B, H, S, D, D, seed, dtype=dt)
        o = ref(q.float(), k.float(), v.float(), causal=causal, softmax_scale=D ** -0.5)
        out[name] = dict(shape=(B, H, S, D, D), causal=causal, seed=seed, dtype=str(dt), o=o.contiguous())

    # sigmoid attention (testing/test.py:519-543)
    ref = extract(tree, source, "test_sigmoid_attention", "ref")
    for name, (B, H, S, D, causal, seed, bias) in {
        "sigmoid_causal": (1, 2, 192, 128, True, 21, -3.0),
        "sigmoid_noncausal_scaled": (1, 2, 256, 128, False, 22, -math.log(256.0)),
    }.items():
        q, k, v = inputs.attention_bshd(B, H, S, D, D, seed)
        qs = q.float() * (D ** -0.5) if "scaled" in name else q.float()
        o = ref(qs, k.float(), v.float(), torch.tensor([bias]), causal=causal)
        out[name] = dict(shape=(B, H, S, D, D), causal=causal, seed=seed, bias=bias, scaled="scaled" in name, o=o.contiguous())

    # relu attention (testing/test.py:599-604); closure reads D from the enclosing scope
    B, H, S, D = 1, 3, 192, 64
    ref = extract(tree, source, "test_relu_attention", "ref", {"D": D})
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 31, k_scale=0.5, v_scale=0.5)
    out["relu"] = dict(shape=(B, H, S, D, D), seed=31, o=ref(q.float(), k.float(), v.float()).contiguous())

    # RetNet retention (testing/test.py:738-747)
    ref = extract(tree, source, "test_retnet_recurrent", "ref")
    B, H, S, Dk, Dv = 1, 8, 192, 64, 128
    q, k, v, _ = inputs.retention_bhsd(B, H, S, Dk, Dv, 41)
    out["retention"] = dict(shape=(B, H, S, Dk, Dv), seed=41, o=ref(q.float(), k.float(), v.float()).contiguous())

    # MLA decode (testing/test.py:807-839)
    ref = extract(tree, source, "test_mla_decode", "ref")
    B, H, S, D, Dv = 2, 16, 384, 576, 512
    q, kv = inputs.mla_inputs(B, H, S, D, Dv, 51)
    o = ref(q[..., :Dv].float(), q[..., Dv:].float(), kv[..., :Dv].float(), kv[..., Dv:].float())
    out["mla"] = dict(shape=(B, H, S, D, Dv), seed=51, o=o.contiguous())

    # gated retention / simple GLA (testing/test.py:436-481), chunk size 64 as the reference test calls it
    ref = extract(tree, source, "test_gated_retention", "naive_chunk_simple_gla", {"Optional": __import__("typing").Optional})
    B, H, S, D, Dv = 1, 4, 200, 64, 128
    q, k, v, g = inputs.gla_inputs(B, H, S, D, Dv, 61)
    out["gla"] = dict(shape=(B, H, S, D, Dv), seed=61, o=ref(q, k, v, g, chunk_size=64)[0].contiguous())

    # Mamba2 SSD (testing/test.py:206-343): the combined reference and the three closures it calls
    helpers = {}
    for name in ("chunk_state_ref", "state_passing_ref", "chunk_scan_ref"):
        helpers[name] = extract(tree, source, "test_mamba2", name, helpers)
    ref = extract(tree, source, "test_mamba2", "ssd_chunk_scan_combined_ref", helpers)
    B, HQ, HK, HV, S, D, Dv = 1, 2, 2, 4, 192, 64, 64
    q, k, v, dt, A = inputs.mamba2_inputs(B, HQ, HK, HV, S, D, Dv, 71)
    # the reference layout is [B,S,H,*]: x = v, B = k, C = q
    o = ref(v.float().transpose(1, 2), dt.transpose(1, 2), A[0], k.float().transpose(1, 2), q.float().transpose(1, 2), chunk_size=64)
    out["mamba2"] = dict(shape=(B, HQ, HK, HV, S, D, Dv), seed=71, o=o.transpose(1, 2).contiguous())

    # MHA decode (testing/test.py:131-148): a few query rows against a longer KV, no mask
    ref = extract(tree, source, "test_softmaxattention_decode", "ref")
    B, H, Sq, KV, D = 2, 4, 3, 320, 64
    g = torch.Generator().manual_seed(81)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, KV, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, KV, H, D, generator=g).to(torch.bfloat16)
    out["mha_decode"] = dict(shape=(B, H, Sq, KV, D, D), seed=81, o=ref(q.float(), k.float(), v.float()).contiguous())

    # block-sparse, variable-length GQA decode (testing/test.py:654-694).  The closure builds two index tensors on
    # device 'cuda'; that literal is replaced by 'cpu', nothing else is touched.
    ref = extract(tree, source, "test_sparse_gqa_decode", "ref_program_torch", edit=lambda seg: seg.replace("'cuda'", "'cpu'"))
    B, H, G, S, D, block = 2, 8, 2, 512, 64, 32
    g = torch.Generator().manual_seed(91)
    q = torch.randn(B, 1, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, G, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, G, D, generator=g).to(torch.bfloat16)
    lens = torch.tensor([S, 300], dtype=torch.int32)
    nblk = S // block
    bmask = torch.rand(B, G, nblk, generator=g) < 0.4
    bmask[:, :, 0] = True   # every (batch, kv head) keeps at least its first block
    o = ref(q.float(), k.float(), v.float(), bmask, lens, S, nblk, block)
    out["sparse_gqa_decode"] = dict(shape=(B, H, G, S, D, D), seed=91, block=block, cache_seqlens=lens, block_mask=bmask,
                                    o=o.contiguous())

    # gradients of softmax MHA: torch autograd through the reference's own closure (testing/test.py:79-104), which is
    # what the reference's test compares its backward kernels with (testing/test.py:106-127); dO is part of the fixture
    ref = extract(tree, source, "test_softmaxattention", "ref")
    for name, (B, H, S, D, causal, seed) in {"softmax_bwd_causal": (1, 2, 160, 128, True, 101),
                                              "softmax_bwd_noncausal": (1, 2, 144, 128, False, 102)}.items():
        q, k, v = inputs.attention_bshd(B, H, S, D, D, seed)
        d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(seed + 1000)).to(torch.bfloat16)
        with torch.enable_grad():
            qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
            o = ref(qf, kf, vf, causal=causal, softmax_scale=D ** -0.5)
            o.backward(d_o.float())
        rec = dict(shape=(B, H, S, D, D), causal=causal, seed=seed, d_o=d_o, o=o.detach().contiguous(),
                   dq=qf.grad.contiguous(), dk=kf.grad.contiguous(), dv=vf.grad.contiguous())
        torch.save(rec, os.path.join(HERE, f"{name}.pt"))
        print(name, tuple(rec["dq"].shape), f"{4 * rec['dq'].numel() * 4 / 1024:.0f} KiB")

    # gradients of sigmoid attention (an elementwise program): autograd through the reference's closure
    # (testing/test.py:519-543) with respect to q, k, v
    ref = extract(tree, source, "test_sigmoid_attention", "ref")
    B, H, S, D, bias = 1, 2, 144, 128, -3.0
    q, k, v = inputs.attention_bshd(B, H, S, D, D, 121)
    d_o = torch.randn(B, S, H, D, generator=torch.Generator().manual_seed(1121)).to(torch.bfloat16)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        o = ref(qf * (D ** -0.5), kf, vf, torch.tensor([bias]), causal=True)
        o.backward(d_o.float())
    rec = dict(shape=(B, H, S, D, D), seed=121, bias=bias, causal=True, d_o=d_o, o=o.detach().contiguous(),
               dq=qf.grad.contiguous(), dk=kf.grad.contiguous(), dv=vf.grad.contiguous())
    torch.save(rec, os.path.join(HERE, "sigmoid_bwd.pt"))
    print("sigmoid_bwd", tuple(rec["dq"].shape))

    # gradients of RetNet retention: autograd through the reference's closure (testing/test.py:738-747)
    ref = extract(tree, source, "test_retnet_recurrent", "ref")
    B, H, S, Dk, Dv = 1, 2, 160, 64, 128
    q, k, v, _ = inputs.retention_bhsd(B, H, S, Dk, Dv, 111)
    d_o = torch.randn(B, H, S, Dv, generator=torch.Generator().manual_seed(1111)).to(torch.bfloat16)
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        o = ref(qf, kf, vf)
        o.float().backward(d_o.float())
    rec = dict(shape=(B, H, S, Dk, Dv), seed=111, d_o=d_o, o=o.detach().float().contiguous(),
               dq=qf.grad.contiguous(), dk=kf.grad.contiguous(), dv=vf.grad.contiguous())
    torch.save(rec, os.path.join(HERE, "retention_bwd.pt"))
    print("retention_bwd", tuple(rec["dv"].shape))

    torch.save(block_mask_goldens(ref_root), os.path.join(HERE, "block_masks.pt"))
    print("block_masks", len(MASK_CASES) * len(MASK_SHAPES), "cases")

    for name, rec in out.items():
        rec["o"] = rec["o"].to(torch.float32)
        torch.save(rec, os.path.join(HERE, f"{name}.pt"))
        print(name, tuple(rec["o"].shape), f"{rec['o'].numel() * 4 / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
