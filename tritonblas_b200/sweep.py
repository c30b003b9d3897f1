"""Selector validation sweeps: the tile / schedule the analytical selector picks against an exhaustive search of the launch
space, and the stream-K grid sweep with last-wave occupancy.

The B200 counterparts of the reference's tools/fp4_selector_efficiency_sweep.py:59-240 (selector pick vs best of all
configurations, "selector efficiency" = best time / picked time) and tools/sweep_grid.py:33-183 (time per sk_grid with
the occupancy of the last tile wave), over this library's launch space: CTA pair {1, 2}, tile width block_n, one or two
accumulators per tile (n_halves), and for stream-K launches the grid.

    python -m tritonblas_b200.sweep --preset baseline --steady --out-csv sweep.csv   # the headline shapes, back to back
    python -m tritonblas_b200.sweep --m 4096 --n 4096 --k 4096 --dtype bf16
    python -m tritonblas_b200.sweep --sk-grid --m 16 --n 28672 --k 8192 --dtype bf16 --min-grid 32 --max-grid 148

Every row: shape, dtype, mode, configuration, measured microseconds (median of cold-L2 repeats), TFLOP/s, whether it is the
selector's pick, the selector's predicted microseconds for its pick, and for grid sweeps the last-wave occupancy.
"""
import argparse
import csv
import sys

import torch

import tritonblas_b200 as tb
from tritonblas_b200 import utils
from tritonblas_b200.bench import do_bench

FP8 = torch.float8_e4m3fn
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp8": FP8, "mxfp4": "mxfp4"}
FIELDS = ["m", "n", "k", "dtype", "mode", "cta_pair", "block_n", "n_halves", "sk_grid", "us", "tflops", "selected",
          "predicted_us", "last_wave_occupancy", "efficiency_vs_best"]

# The shapes the headline metric is quoted on: (m, n, k, dtype, stream-K)
BASELINE = [
    (8192, 8192, 8192, "bf16", False),
    (4096, 4096, 4096, "bf16", False),
    (4864, 8192, 4160, "bf16", False),
    (1024, 1024, 1024, "fp16", False),
    (4096, 28672, 8192, "fp8", False),
    (256, 28672, 8192, "fp8", False),
    (128, 28672, 8192, "bf16", True),
    (16, 28672, 8192, "bf16", True),
    (16, 28672, 8192, "fp8", True),
    (8192, 8192, 8192, "mxfp4", False),
]


class Problem:
    """Operands of one shape and a launch function that takes a forced configuration."""

    def __init__(self, m, n, k, dtype, streamk):
        self.m, self.n, self.k, self.dtype, self.streamk = m, n, k, dtype, streamk
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev).manual_seed(m + n + k)
        self.c = torch.empty(m, n, dtype=torch.bfloat16 if dtype in ("fp8", "mxfp4") else DTYPES[dtype], device=dev)
        if dtype == "mxfp4":
            a = torch.randn(m, k, generator=g, device=dev, dtype=torch.bfloat16)
            b = torch.randn(n, k, generator=g, device=dev, dtype=torch.bfloat16)
            self.qa, self.sa = utils.dynamic_mxfp4_quant(a, scale_atoms=True)
            self.qb, self.sb = utils.dynamic_mxfp4_quant(b, scale_atoms=True)
            return
        a = torch.randn(m, k, generator=g, device=dev, dtype=torch.bfloat16) * (1.0 if dtype == "fp8" else 0.02)
        b = torch.randn(n, k, generator=g, device=dev, dtype=torch.bfloat16) * 0.02
        if dtype == "fp8":
            self.a, self.a_s = utils.quantize_fp8_rows(a)
            bq, self.b_s = utils.quantize_fp8_rows(b)
            self.b = bq.T
        else:
            self.a, self.b = a.to(DTYPES[dtype]), b.to(DTYPES[dtype]).T
            self.a_s = self.b_s = None

    def selector(self):
        if self.dtype == "mxfp4":
            return tb.OrigamiMatmulSelector(self.m, self.n, self.k, "f4", "f4", torch.bfloat16, self.c.device, mx_block_size=32)
        dt = DTYPES[self.dtype]
        return tb.OrigamiMatmulSelector(self.m, self.n, self.k, dt, dt, self.c.dtype, self.c.device, streamk=self.streamk)

    def candidates(self):
        """(cta_pair, block_n, n_halves) the kernels accept for this problem."""
        if self.dtype == "mxfp4":
            return [(p, bn, 1) for p in (1, 2) for bn in (64, 128, 192)]
        out = []
        swapped = self.selector()._cfg.swap_ab == 1
        n_eff = self.m if swapped else self.n
        m_eff = self.n if swapped else self.m
        for pair in (1, 2):
            if pair == 2 and m_eff <= 128:
                continue
            for bn in (32, 64, 128, 256):
                if (bn // pair) < 16 or (bn >= 2 * n_eff and bn > 32):
                    continue
                out.append((pair, bn, 1))
                if bn == 256 and not self.streamk and n_eff >= 2 * bn:
                    out.append((pair, bn, 2))
        return out

    def launcher(self, pair, bn, halves, sk_grid=None):
        if self.dtype == "mxfp4":
            return lambda: tb.matmul_fp4(self.qa, self.qb, self.c, self.sa, self.sb, block_m=128 * pair, block_n=bn)
        sel = self.selector()
        if pair is not None:
            sel.override(cta_pair=pair, block_n=bn, n_halves=halves)
        cfg = tb.matmul_preamble(sel)
        if self.a_s is not None:
            if self.streamk:
                return lambda: tb.streamk_matmul_lt(self.a, self.b, self.c, sel, cfg, sk_grid=sk_grid, a_scale=self.a_s,
                                                    b_scale=self.b_s, quantized=True)
            return lambda: tb.matmul_a8w8_lt(self.a, self.b, self.a_s, self.b_s, self.c, sel, cfg)
        if self.streamk:
            return lambda: tb.streamk_matmul_lt(self.a, self.b, self.c, sel, cfg, sk_grid=sk_grid)
        return lambda: tb.matmul_lt(self.a, self.b, self.c, sel, cfg)


_MODE = {"steady": False}


def _time_us(fn, warmup, repeats):
    """Microseconds per launch. Cold mode: every launch on its own after an L2 flush (the reference's do_bench; for launches
    of tens of microseconds this includes the host's launch latency, and the chip is cool, so clocks are high). Steady mode:
    launches back to back for at least a quarter of a second, which is how a training or serving loop meets the kernel: the
    chip sits at its power limit and what counts is work per joule."""
    if not _MODE["steady"]:
        return 1e3 * do_bench(fn, n_warmup=warmup, n_repeat=repeats, return_mode="median")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        fn()
    e1.record()
    torch.cuda.synchronize()
    n = max(repeats, min(5000, int(250.0 / max(e0.elapsed_time(e1) / 10, 1e-3))))
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return 1e3 * e0.elapsed_time(e1) / n


def sweep_tiles(m, n, k, dtype, streamk, warmup=5, repeats=30, out=sys.stdout):
    """Every accepted (cta_pair, block_n, n_halves) of one problem, timed; the selector's own pick marked."""
    prob = Problem(m, n, k, dtype, streamk)
    sel = prob.selector()
    cfg = sel._cfg
    pick = (2 if cfg.cta_pair == 2 else 1, cfg.block_n, max(cfg.n_halves, 1) if not streamk and dtype != "mxfp4" else 1)
    flops = 2.0 * m * n * k
    rows = []
    for pair, bn, halves in prob.candidates():
        try:
            us = _time_us(prob.launcher(pair, bn, halves), warmup, repeats)
        except tb.TritonBlasError as exc:      # a width the kernel refuses for this layout
            print(f"  skip pair={pair} bn={bn} halves={halves}: {exc}", file=out)
            continue
        rows.append({"m": m, "n": n, "k": k, "dtype": dtype, "mode": "streamk" if streamk else "persistent",
                     "cta_pair": pair, "block_n": bn, "n_halves": halves, "sk_grid": cfg.sk_grid if streamk else "",
                     "us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "selected": int((pair, bn, halves) == pick),
                     "predicted_us": round(sel.predicted_us, 2) if (pair, bn, halves) == pick else "", "last_wave_occupancy": ""})
    best = min(r["us"] for r in rows)
    for r in rows:
        r["efficiency_vs_best"] = round(best / r["us"], 3)
    picked = [r for r in rows if r["selected"]]
    eff = picked[0]["efficiency_vs_best"] if picked else float("nan")
    print(f"{dtype} {m}x{n}x{k} {'stream-K' if streamk else 'persistent'}: selector picks pair={pick[0]} bn={pick[1]} "
          f"halves={pick[2]} -> {picked[0]['us'] if picked else '?'} us (predicted {sel.predicted_us:.1f}), best {best} us, "
          f"selector efficiency {100 * eff:.1f} %", file=out)
    return rows, eff


def sweep_sk_grid(m, n, k, dtype, min_grid, max_grid, step=1, warmup=5, repeats=30, out=sys.stdout):
    """Stream-K time per grid size with the occupancy of the last wave of tiles (tools/sweep_grid.py:162-183)."""
    prob = Problem(m, n, k, dtype, True)
    sel = prob.selector()
    cfg = sel._cfg
    pair = 2 if cfg.cta_pair == 2 else 1
    swapped = cfg.swap_ab == 1
    tiles = -(-(n if swapped else m) // cfg.block_m) * -(-(m if swapped else n) // cfg.block_n)
    flops = 2.0 * m * n * k
    rows = []
    for grid in range(min_grid, min(max_grid, cfg.num_sms // pair) + 1, step):
        us = _time_us(prob.launcher(None, None, None, sk_grid=grid), warmup, repeats)
        rem = tiles % grid
        rows.append({"m": m, "n": n, "k": k, "dtype": dtype, "mode": "streamk", "cta_pair": pair, "block_n": cfg.block_n,
                     "n_halves": 1, "sk_grid": grid, "us": round(us, 2), "tflops": round(flops / us / 1e6, 1),
                     "selected": int(grid == cfg.sk_grid), "predicted_us": round(sel.predicted_us, 2) if grid == cfg.sk_grid else "",
                     "last_wave_occupancy": round(rem / grid, 3) if rem else 1.0})
    best = min(r["us"] for r in rows)
    for r in rows:
        r["efficiency_vs_best"] = round(best / r["us"], 3)
    top = sorted(rows, key=lambda r: r["us"])[:10]
    print(f"{dtype} {m}x{n}x{k} stream-K, {tiles} tiles of {cfg.block_m}x{cfg.block_n}; selector grid {cfg.sk_grid}", file=out)
    for r in top:
        print(f"  sk_grid {r['sk_grid']:4d}  {r['us']:9.2f} us  {r['tflops']:8.1f} TFLOP/s  last wave {100 * r['last_wave_occupancy']:5.1f} %"
              f"{'  <- selector' if r['selected'] else ''}", file=out)
    picked = [r for r in rows if r["selected"]]
    return rows, (picked[0]["efficiency_vs_best"] if picked else float("nan"))


def write_csv(path, rows):
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=FIELDS)
        w.writeheader()
        for r in rows:
            w.writerow({k: r.get(k, "") for k in FIELDS})


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--preset", choices=["baseline"], help="sweep the headline shapes")
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    ap.add_argument("--streamk", action="store_true")
    ap.add_argument("--sk-grid", action="store_true", help="sweep the stream-K grid instead of the tile space")
    ap.add_argument("--min-grid", type=int, default=16)
    ap.add_argument("--max-grid", type=int, default=148)
    ap.add_argument("--grid-step", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=30)
    ap.add_argument("--out-csv")
    ap.add_argument("--steady", action="store_true",
                    help="time launches back to back (>= 0.25 s per configuration) instead of one cold launch at a time")
    args = ap.parse_args(argv)
    _MODE["steady"] = bool(args.steady)
    rows, effs = [], []
    if args.preset == "baseline":
        for m, n, k, dt, sk in BASELINE:
            r, e = sweep_tiles(m, n, k, dt, sk, args.warmup, args.repeats)
            rows += r
            effs.append(e)
    elif args.sk_grid:
        r, e = sweep_sk_grid(args.m, args.n, args.k, args.dtype, args.min_grid, args.max_grid, args.grid_step, args.warmup,
                             args.repeats)
        rows += r
        effs.append(e)
    else:
        if not (args.m and args.n and args.k):
            ap.error("give --preset baseline, or --m --n --k")
        r, e = sweep_tiles(args.m, args.n, args.k, args.dtype, args.streamk, args.warmup, args.repeats)
        rows += r
        effs.append(e)
    print(f"selector efficiency: min {100 * min(effs):.1f} %, mean {100 * sum(effs) / len(effs):.1f} % over {len(effs)} problem(s)")
    if args.out_csv:
        write_csv(args.out_csv, rows)
    return rows, effs


if __name__ == "__main__":
    main()
