"""``do_bench``: CUDA-event timing of a launch function with a cold L2 before every repeat; same arguments, defaults and
return modes as the reference's (include/tritonblas/bench.py:64-131).

``reset_fn`` and ``preamble_fn`` run before every invocation and are not timed. Between invocations a buffer larger
than the 126 MB L2 is overwritten, so every repeat reads its operands from HBM.
"""
import math
import statistics

import torch

_FLUSH_BYTES = 512 * 1024 * 1024
_flush_buffers = {}


def _flush_l2():
    dev = torch.cuda.current_device()
    buf = _flush_buffers.get(dev)
    if buf is None:
        buf = _flush_buffers[dev] = torch.empty(_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda")
    buf.add_(1)          # read-modify-write of every line: evicts whatever the previous launch left in L2


def _quantiles(times, qs):
    ordered = sorted(times)
    out = []
    for q in qs:
        if not 0 <= q <= 1:
            raise ValueError("Quantiles must be in the range [0, 1]")
        pos = q * (len(ordered) - 1)
        lo, hi = math.floor(pos), math.ceil(pos)
        out.append(ordered[lo] + (ordered[hi] - ordered[lo]) * (pos - lo))
    return out


def do_bench(fn, reset_fn=lambda: None, preamble_fn=lambda: None, n_warmup=25, n_repeat=100, quantiles=None,
             return_mode="mean"):
    """Milliseconds per call of ``fn``: ``return_mode`` of "mean", "min", "max", "median" or "all" (the list), or the
    requested ``quantiles`` (a single value when one quantile is asked for)."""
    if return_mode not in ("mean", "min", "max", "median", "all"):
        raise ValueError(f"unknown return_mode {return_mode!r}")
    torch.cuda.synchronize()
    preamble_fn()
    reset_fn()
    fn()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(n_warmup + n_repeat):
        torch.cuda.synchronize()
        reset_fn()
        preamble_fn()
        _flush_l2()
        torch.cuda.synchronize()
        if i < n_warmup:
            fn()
            continue
        starts[i - n_warmup].record()
        fn()
        stops[i - n_warmup].record()
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    if quantiles is not None:
        q = _quantiles(times, quantiles)
        return q[0] if len(q) == 1 else q
    if return_mode == "all":
        return times
    return {"mean": statistics.mean, "min": min, "max": max, "median": statistics.median}[return_mode](times)
