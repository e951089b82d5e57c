"""Timing and comparison helpers with the signatures the reference's test
suite imports (``from benchmark.bench_utils import print_debug, assert_close,
do_bench``; attention_engine/benchmark/bench_utils.py:14-99, :133-173,
:200-225).  No plotting dependency; vendor-library comparison harnesses of the
reference are not provided."""

from __future__ import annotations

import statistics

import torch

L2_FLUSH_BYTES = 256 * 1024 * 1024  # larger than the 126 MB L2 of a B200


def do_bench(fn, warmup=25, rep=100, _n_warmup=0, _n_repeat=0, grad_to_none=None,
             quantiles=None, fast_flush=True, return_mode="mean", flush_l2=True):
    """Time ``fn`` with CUDA events on the current stream, in milliseconds.

    ``warmup``/``rep`` are time budgets in ms (converted to iteration counts
    from a 5-launch estimate) unless ``_n_warmup``/``_n_repeat`` give counts.
    Each timed launch has its own event pair; with ``flush_l2`` a 256 MB buffer
    is overwritten before each launch (outside the timed pair) so inputs are
    not served from L2.  ``return_mode``: mean | median | min | max.  With
    ``quantiles`` a list of those quantiles is returned instead."""
    assert return_mode in ("min", "max", "mean", "median")
    fn()
    torch.cuda.synchronize()
    cache = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda") if flush_l2 else None

    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        fn()
    e1.record()
    torch.cuda.synchronize()
    estimate_ms = max(e0.elapsed_time(e1) / 5, 1e-3)
    n_warmup = _n_warmup if _n_warmup > 0 else max(3, int(warmup / estimate_ms))
    n_repeat = _n_repeat if _n_repeat > 0 else max(1, int(rep / estimate_ms))
    n_warmup = min(n_warmup, 1000)
    n_repeat = min(n_repeat, 2000)

    for _ in range(n_warmup):
        fn()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_repeat):
        if grad_to_none is not None:
            for x in grad_to_none:
                x.grad = None
        if cache is not None:
            cache.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    if quantiles is not None:
        t = torch.tensor(times, dtype=torch.float64)
        return torch.quantile(t, torch.tensor(quantiles, dtype=torch.float64)).tolist()
    return {"min": min, "max": max, "mean": statistics.fmean, "median": statistics.median}[return_mode](times)


def assert_close(actual, expected, rtol: float = 1e-5, atol: float = 1e-8, equal_nan: bool = False,
                 mismatch_ratio: float = 0.0, msg: str | None = None):
    """Like ``torch.testing.assert_close`` but tolerating a fraction
    ``mismatch_ratio`` (0..1) of elements outside ``atol + rtol*|expected|``."""
    actual = torch.as_tensor(actual)
    expected = torch.as_tensor(expected).to(actual.device)
    ok = torch.isclose(actual.float(), expected.float(), rtol=rtol, atol=atol, equal_nan=equal_nan)
    total = ok.numel()
    bad = int((~ok).sum().item())
    ratio = bad / max(total, 1)
    if ratio > mismatch_ratio:
        raise AssertionError(msg or (
            f"Mismatch ratio {ratio:.6f} exceeds allowed threshold {mismatch_ratio}.\n"
            f"Mismatched elements: {bad}/{total}"))


def print_debug(o, O_ref, rtol=1e-3, atol=1e-3, save_file=True):
    """Print how many elements of ``o`` fall outside ``atol + rtol*|O_ref|`` and
    where the largest excess is.  Returns the count."""
    o = torch.as_tensor(o).float()
    O_ref = torch.as_tensor(O_ref).float().to(o.device)
    diff = (o - O_ref).abs()
    over = diff > (atol + rtol * O_ref.abs())
    n_over = int(over.sum().item())
    total = o.numel()
    print(f"{n_over} elements exceed tolerance.")
    print(f"{100.0 * n_over / max(total, 1):.2f}% of the elements exceed tolerance.")
    print(f"Total elements: {total}, Exceed tolerance elements: {n_over}")
    if n_over:
        masked = torch.where(over, diff, torch.zeros_like(diff))
        flat = int(masked.argmax().item())
        idx = tuple(int(i) for i in torch.unravel_index(torch.tensor(flat), o.shape))
        print(f"Max exceed diff: {masked.flatten()[flat].item()} at index {idx}")
        print(f"  got {o[idx].item()}  expected {O_ref[idx].item()}")
    print(f"max abs diff {diff.max().item():.6g}  mean abs diff {diff.mean().item():.6g}")
    return n_over


def error_stats(actual, expected) -> dict:
    """max-abs and mean-abs error of ``actual`` against ``expected`` (both cast to fp32)."""
    a = torch.as_tensor(actual).float().cpu()
    e = torch.as_tensor(expected).float().cpu()
    d = (a - e).abs()
    return {"max_abs": float(d.max()), "mean_abs": float(d.mean())}
