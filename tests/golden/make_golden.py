"""Generates tests/golden/*.pt: outputs of the REFERENCE's own PyTorch reference
closures on seeded inputs.  Run in a container that has the reference checkout:

    python tests/golden/make_golden.py [/path/to/reference]

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


def extract(tree, source, outer: str, inner: str, extra_globals=None):
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == outer:
            for sub in ast.walk(node):
                if isinstance(sub, ast.FunctionDef) and sub.name == inner and sub is not node:
                    seg = ast.get_source_segment(source, sub)
                    import textwrap
                    ns = {"torch": torch, "F": F, "rearrange": rearrange, "einsum": einsum, "repeat": repeat,
                          "math": math}
                    ns.update(extra_globals or {})
                    exec(textwrap.dedent(seg), ns)
                    return ns[inner]
    raise KeyError(f"{outer}.{inner} not found")


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
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

    for name, rec in out.items():
        rec["o"] = rec["o"].to(torch.float32)
        torch.save(rec, os.path.join(HERE, f"{name}.pt"))
        print(name, tuple(rec["o"].shape), f"{rec['o'].numel() * 4 / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
