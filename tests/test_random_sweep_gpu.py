"""Seeded random sweep over shapes, dtypes, masks and head layouts of the three kernel families against
the CPU oracle (same tolerances as the targeted tests).  Cheap cases only: the whole sweep runs in seconds."""

import random

import pytest
import torch

from examples_b200 import programs
from attn_engine import AttentionEngine
from attn_engine.linear_attn_engine import linear_attention_forward
from attn_engine.mla import mla_decode_forward
from core import CustomIO, meta_tensor
from core.native import lib
from oracle import reference_math as rm

pytestmark = pytest.mark.gpu


def _close(kind, cfg, o, want, max_abs=2e-2, mean_abs=2e-3, rel=None):
    assert lib.last_device_status() == 0, (kind, cfg)
    o = o.float().cpu()
    assert torch.isfinite(o).all(), (kind, cfg)
    if rel is None:
        d = (o - want.float()).abs()
        assert d.max().item() <= max_abs and d.mean().item() <= mean_abs, (kind, cfg, d.max().item(), d.mean().item())
    else:
        assert ((o - want).norm() / want.norm()).item() <= rel, (kind, cfg)


def _attention_case(rnd, g, kind):
    D = rnd.choice([64, 128])
    dt = rnd.choice([torch.bfloat16, torch.float16])
    B, Hkv = rnd.randint(1, 3), rnd.randint(1, 4)
    H = Hkv * (rnd.choice([1, 1, 2, 4]) if kind in ("gqa", "decode") else 1)
    Skv = rnd.choice([1, 63, 128, 129, 255, 256, 257, 500, 1000, 1537])
    Sq = Skv if kind != "decode" else rnd.choice([1, 2, 17, 128, 300])
    q = torch.randn(B, Sq, H, D, generator=g).to(dt)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(dt)
    v = torch.randn(B, Skv, Hkv, D, generator=g).to(dt)
    qi, ki = torch.arange(Sq).view(-1, 1), torch.arange(Skv).view(1, -1)
    if kind == "band":
        left, right = rnd.choice([0, 1, 5, 64, 127, 128, 200, 10 ** 9]), rnd.choice([0, 0, 3, 100, 10 ** 9])
        mask_mod = lambda b, h, qq, kk: (qq - kk <= left) & (kk - qq <= right)   # noqa: E731
        keep = mask_mod(0, 0, qi, ki)
    elif kind == "decode" or rnd.random() < 0.5:
        mask_mod, keep = None, torch.ones(Sq, Skv, dtype=torch.bool)
    else:
        mask_mod, keep = programs.causal, ki <= qi
    scale = D ** -0.5
    meta = (meta_tensor(B, H, Sq, D, dtype=dt), meta_tensor(B, Hkv, Skv, D, dtype=dt), meta_tensor(B, Hkv, Skv, D, dtype=dt))
    e = AttentionEngine(meta, CustomIO({}), score_mod=lambda s, c, b, h, qq, kk: s * scale, mask_mod=mask_mod,
                        online_func=programs.NaturalSoftmax())
    o = e(q.cuda(), k.cuda(), v.cuda())
    _close(kind, (B, H, Hkv, Sq, Skv, D, dt), o, rm.softmax_attention(q, k, v, softmax_scale=scale, keep=keep))


def _mla_case(rnd, g):
    B, H = rnd.randint(1, 5), rnd.choice([16, 64, 128, 256])
    S = rnd.choice([1, 64, 129, 500, 1024, 3000])
    dt = rnd.choice([torch.bfloat16, torch.float16])
    splits = rnd.choice([None, 1, 2, 3])
    if splits and splits > 1 and (S + 127) // 128 < 4 * splits:
        splits = 1
    q = torch.randn(B, 1, H, 576, generator=g).to(dt)
    kv = torch.randn(B, S, 1, 576, generator=g).to(dt)
    lens = [rnd.randint(1, S) for _ in range(B)] if rnd.random() < 0.5 else None
    o, _ = mla_decode_forward(q.cuda(), kv.cuda(), 512, 576 ** -0.5, num_splits=splits,
                              cache_seqlens=None if lens is None else torch.tensor(lens, dtype=torch.int32, device="cuda"))
    want = torch.cat([rm.mla_decode(q[b:b + 1, ..., :512], q[b:b + 1, ..., 512:], kv[b:b + 1, :(S if lens is None else lens[b]), :, :512],
                                    kv[b:b + 1, :(S if lens is None else lens[b]), :, 512:]) for b in range(B)])
    _close("mla", (B, H, S, dt, splits, lens), o.reshape(B, 1, H, 512), want)


def _linear_case(rnd, g):
    B, H = rnd.randint(1, 2), rnd.randint(1, 4)
    S = rnd.choice([1, 100, 128, 129, 400, 1000])
    Dk, Dv = rnd.choice([64, 128, 256]), rnd.choice([64, 128, 256, 384])
    dt = rnd.choice([torch.bfloat16, torch.float16])
    q = torch.randn(B, H, S, Dk, generator=g).to(dt)
    k = (torch.randn(B, H, S, Dk, generator=g) * Dk ** -0.5).to(dt)
    v = torch.randn(B, H, S, Dv, generator=g).to(dt)
    log_decay = -torch.rand(B, H, S, generator=g) * rnd.choice([0.01, 0.1, 1.0, 4.0])
    o = linear_attention_forward(q.cuda(), k.cuda(), v.cuda(), log_decay.cuda(), q_scale=Dk ** -0.5)
    _close("linear", (B, H, S, Dk, Dv, dt), o, rm.decayed_linear_attention(q, k, v, log_decay, scale=Dk ** -0.5), rel=1e-2)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_sweep(seed):
    rnd = random.Random(seed)
    for _ in range(25):
        kind = rnd.choice(["softmax", "softmax", "band", "gqa", "decode", "mla", "linear"])
        g = torch.Generator().manual_seed(rnd.randrange(1 << 30))
        if kind == "mla":
            _mla_case(rnd, g)
        elif kind == "linear":
            _linear_case(rnd, g)
        else:
            _attention_case(rnd, g, kind)


def _grad_close(kind, cfg, got, want, frac_max=2e-2, frac_mean=3e-3):
    """Gradients (16-bit against fp32): max-abs 2e-2 of the expected tensor's largest value, mean-abs 3e-3 of 1.5 x its
    spread, each at least 1 (tests/test_bwd_gpu.py and tests/test_linear_bwd_gpu.py say why the scales are needed)."""
    got = got.float().cpu()
    assert torch.isfinite(got).all(), (kind, cfg)
    d = (got - want.float()).abs()
    assert d.max().item() <= frac_max * max(1.0, want.abs().max().item()), (kind, cfg, d.max().item(), want.abs().max().item())
    assert d.mean().item() <= frac_mean * max(1.0, 1.5 * want.std().item()), (kind, cfg, d.mean().item(), want.std().item())


def _attention_backward_case(rnd, g):
    D = rnd.choice([64, 128])
    Dv = D * rnd.choice([1, 1, 2]) if D == 128 else D      # the forward covers dim_v = k x 128 only with dim_qk 128
    dt = rnd.choice([torch.bfloat16, torch.float16])
    B, Hkv = rnd.randint(1, 2), rnd.randint(1, 3)
    H = Hkv * rnd.choice([1, 1, 2])
    Sq = rnd.choice([100, 128, 257, 384, 700])
    Skv = Sq if rnd.random() < 0.7 else rnd.choice([200, 512, 900])
    mask = rnd.choice(["none", "causal", "band"]) if Sq == Skv else rnd.choice(["none", "band"])
    q = torch.randn(B, Sq, H, D, generator=g).to(dt)
    k = torch.randn(B, Skv, Hkv, D, generator=g).to(dt)
    v = torch.randn(B, Skv, Hkv, Dv, generator=g).to(dt)
    d_o = torch.randn(B, Sq, H, Dv, generator=g).to(dt)
    qi, ki = torch.arange(Sq).view(-1, 1), torch.arange(Skv).view(1, -1)
    left, right = lib.MASK_OPEN, lib.MASK_OPEN
    if mask == "causal":
        keep, kind_code = ki <= qi, lib.MASK_CAUSAL
    elif mask == "band":
        left = rnd.choice([0, 5, 64, 127, 200, lib.MASK_OPEN])
        right = rnd.choice([0, 0, 3, 100, lib.MASK_OPEN]) if Sq == Skv else rnd.choice([Skv, lib.MASK_OPEN])
        keep, kind_code = (ki >= qi - left) & (ki <= qi + right), lib.MASK_BAND
    else:
        keep, kind_code = torch.ones(Sq, Skv, dtype=torch.bool), lib.MASK_NONE
    scale = D ** -0.5
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        rm.softmax_attention(qf, kf, vf, False, scale, keep=keep).backward(d_o.float())
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty((B, Sq, H, Dv), dtype=dt, device="cuda")
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device="cuda")
    lib.parallel_fwd(lib.fill_parallel_args(qc, kc, vc, o, mask_kind=kind_code, mask_band=(left, right), functor=lib.FUNCTOR_SOFTMAX,
                                            fparams=(scale,), final_rowscales=[lse]))
    dq, dk, dv = lib.softmax_bwd(qc, kc, vc, o, lse, d_o.cuda(), scale, kind_code, (left, right))
    torch.cuda.synchronize()
    cfg = (B, H, Hkv, Sq, Skv, D, Dv, dt, mask, left, right)
    assert lib.last_device_status() == 0, cfg
    for got, want, what in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
        _grad_close("attention backward " + what, cfg, got, want)


def _linear_backward_case(rnd, g):
    from attn_engine.linear_attn_engine import linear_attention_backward
    B, H = rnd.randint(1, 2), rnd.randint(1, 3)
    S = rnd.choice([100, 128, 257, 400])
    Dk, Dv = rnd.choice([64, 128, 256]), rnd.choice([128, 256, 384, 512])
    dt = rnd.choice([torch.bfloat16, torch.float16])
    q = torch.randn(B, H, S, Dk, generator=g).to(dt)
    k = (torch.randn(B, H, S, Dk, generator=g) * Dk ** -0.5).to(dt)
    v = torch.randn(B, H, S, Dv, generator=g).to(dt)
    d_o = torch.randn(B, H, S, Dv, generator=g).to(dt)
    log_decay = -torch.rand(B, H, S, generator=g) * rnd.choice([0.02, 0.1, 0.5])
    with_dg = rnd.random() < 0.5
    want = rm.decayed_linear_attention_grads(q, k, v, log_decay, d_o, scale=Dk ** -0.5, with_decay=with_dg)
    got = linear_attention_backward(q.cuda(), k.cuda(), v.cuda(), log_decay.cuda(), d_o.cuda(), q_scale=Dk ** -0.5, need_dg=with_dg)
    torch.cuda.synchronize()
    cfg = (B, H, S, Dk, Dv, dt, with_dg)
    assert lib.last_device_status() == 0, cfg
    for gt, w, what in zip(got, want, ("dq", "dk", "dv", "dg")):
        if what == "dg":    # a running sum of differences of sums: looser (tests/test_linear_bwd_gpu.py::check_decay_grad)
            _grad_close("linear backward dg", cfg, gt, w, frac_max=1e-1, frac_mean=2e-2)
        else:
            _grad_close("linear backward " + what, cfg, gt, w)


def _general_mask_backward_case(rnd, g):
    """A mask_mod with holes (not a band) through the engine: keep bits + tile bitmaps in the backward."""
    D = rnd.choice([64, 128])
    dt = rnd.choice([torch.bfloat16, torch.float16])
    B, H, S = rnd.randint(1, 2), rnd.randint(1, 3), rnd.choice([200, 384, 640, 900])
    a, b_, c = rnd.choice([32, 64, 100, 200]), rnd.choice([48, 96, 128, 300]), rnd.choice([2, 3, 4])
    causal_too = rnd.random() < 0.5

    def mask_mod(b, h, q_idx, kv_idx):
        m = torch.logical_or(q_idx == kv_idx, ((q_idx // a) + (kv_idx // b_)) % c == 0)
        return torch.logical_and(m, q_idx >= kv_idx) if causal_too else m
    q = torch.randn(B, S, H, D, generator=g).to(dt)
    k = torch.randn(B, S, H, D, generator=g).to(dt)
    v = torch.randn(B, S, H, D, generator=g).to(dt)
    d_o = torch.randn(B, S, H, D, generator=g).to(dt)
    keep = mask_mod(0, 0, torch.arange(S).view(-1, 1), torch.arange(S).view(1, -1))
    scale = D ** -0.5
    with torch.enable_grad():
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        rm.softmax_attention(qf, kf, vf, False, scale, keep=keep).backward(d_o.float())
    meta = (meta_tensor(B, H, S, D, dtype=dt), meta_tensor(B, H, S, D, dtype=dt), meta_tensor(B, H, S, D, dtype=dt))
    e = AttentionEngine(meta, CustomIO({}), score_mod=lambda s_, c_, b, h, qq, kk: s_ * scale, mask_mod=mask_mod,
                        online_func=programs.NaturalSoftmax())
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    e(qc, kc, vc).backward(d_o.cuda())
    torch.cuda.synchronize()
    cfg = (B, H, S, D, dt, a, b_, c, causal_too)
    assert lib.last_device_status() == 0, cfg
    for got, want, what in ((qc.grad, qf.grad, "dq"), (kc.grad, kf.grad, "dk"), (vc.grad, vf.grad, "dv")):
        _grad_close("general-mask backward " + what, cfg, got, want)


@pytest.mark.parametrize("seed", [21, 22])
def test_random_sweep_backward(seed):
    """The backward kernels over random shapes, dtypes, head groups, ragged lengths and masks (none, causal, bands)."""
    rnd = random.Random(seed)
    for _ in range(14):
        g = torch.Generator().manual_seed(rnd.randrange(1 << 30))
        r = rnd.random()
        if r < 0.5:
            _attention_backward_case(rnd, g)
        elif r < 0.7:
            _general_mask_backward_case(rnd, g)
        else:
            _linear_backward_case(rnd, g)
