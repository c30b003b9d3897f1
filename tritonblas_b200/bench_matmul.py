"""YAML-driven GEMM benchmark that writes one CSV row per shape.

Same inputs and outputs as the reference's benchmark driver (benchmarks/tritonblas_matmul.py:118-301): a YAML list of
cases ``{m, n, k, in_dtype, out_dtype, transA, transB}``, the ``*_lt`` entry points with a selector and a pre-allocated
``MatmulConfig`` per case, and a CSV with the columns m, n, k, mnk, macro_tile, bytes, flops, tritonblas_gflops, a_type,
b_type, c_type, d_type, compute_type, in_dtype, out_dtype, init_type, transA, transB, us, alpha, beta, mode (plus
active_cus when an SM sweep is asked for). Timing is by CUDA events on the current stream; between repeats a buffer
larger than L2 is overwritten so every repeat starts cold, as the reference's ``do_bench`` does.

    python -m tritonblas_b200.bench_matmul --input-yaml tritonblas_b200/shapes/baseline.yaml --output-csv out.csv
    python -m tritonblas_b200.bench_matmul --input-yaml shapes.yaml --work-stealing --cu-sweep 148,116,84 --output-csv sweep.csv
"""
import argparse
import csv
import random
import statistics

import torch

import tritonblas_b200 as tb
from tritonblas_b200 import utils
from tritonblas_b200.bench import do_bench

_DTYPES = {"fp16": torch.float16, "float16": torch.float16, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
           "fp32": torch.float32, "float32": torch.float32, "fp8": torch.float8_e4m3fn, "fp8e4m3": torch.float8_e4m3fn,
           "fp8_e4m3": torch.float8_e4m3fn, "fp8_e5m2": torch.float8_e5m2, "int8": torch.int8}

CSV_FIELDS = ["m", "n", "k", "mnk", "macro_tile", "bytes", "flops", "tritonblas_gflops", "a_type", "b_type", "c_type",
              "d_type", "compute_type", "in_dtype", "out_dtype", "init_type", "transA", "transB", "us", "alpha", "beta",
              "mode"]


def str_to_dtype(name):
    key = str(name).replace("torch.", "").lower()
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}")
    return _DTYPES[key]


def bench_case(case, init_type="randn", enable_streamk=False, work_stealing=False, active_cus=None, check=False,
               n_warmup=20, n_repeat=100):
    m, n, k = int(case["m"]), int(case["n"]), int(case["k"])
    in_dtype, out_dtype = str_to_dtype(case["in_dtype"]), str_to_dtype(case["out_dtype"])
    trans_a, trans_b = case.get("transA", "T"), case.get("transB", "T")
    inputs = utils.generate_matmul_inputs(m, n, k, in_dtype, out_dtype, trans_a, trans_b, init_type)
    selector = tb.OrigamiMatmulSelector(m, n, k, inputs.A.dtype, inputs.B.dtype, inputs.C.dtype, inputs.A.device,
                                        streamk=enable_streamk, active_cus=active_cus)
    cfg = tb.matmul_preamble(selector)
    if inputs.is_quantized:
        def launch():
            tb.matmul_a8w8_lt(inputs.A, inputs.B, inputs.scaleA, inputs.scaleB, inputs.C, selector, cfg, enable_streamk,
                              work_stealing=work_stealing)
    else:
        def launch():
            tb.matmul_lt(inputs.A, inputs.B, inputs.C, selector, cfg, enable_streamk, work_stealing=work_stealing)
    ms = do_bench(launch, n_warmup=n_warmup, n_repeat=n_repeat, return_mode="median")
    tb.raise_on_device_failure()
    if check:
        a32, b32 = inputs.A.float(), inputs.B.float()
        ref = a32 @ b32
        if inputs.is_quantized:
            ref = ref * inputs.scaleA.float().view(-1, 1) * inputs.scaleB.float().view(1, -1)
        err = (inputs.C.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        if not err <= 0.05 * scale + 0.5:
            raise AssertionError(f"m={m} n={n} k={k}: max error {err} against reference magnitude {scale}")
    nbytes = sum(t.numel() * t.element_size() for t in (inputs.A, inputs.B, inputs.C, inputs.scaleA, inputs.scaleB)
                 if t is not None)
    mode = "work_stealing" if work_stealing and not enable_streamk else "streamk" if enable_streamk else "persistent"
    row = {
        "m": m, "n": n, "k": k, "mnk": m * n * k,
        "macro_tile": f"{selector.block_m}x{selector.block_n * max(selector.config_for(False, False).n_halves, 1)}x{selector.block_k}",
        "bytes": nbytes, "flops": 2 * m * n * k * 1e-12, "tritonblas_gflops": 2 * m * n * k * 1e-9 / (ms * 1e-3),
        "a_type": str(inputs.A.dtype), "b_type": str(inputs.B.dtype), "c_type": str(inputs.C.dtype),
        "d_type": str(inputs.C.dtype), "compute_type": str(inputs.C.dtype), "in_dtype": str(in_dtype),
        "out_dtype": str(out_dtype), "init_type": init_type, "transA": str(trans_a), "transB": str(trans_b),
        "us": ms * 1000.0, "alpha": 1, "beta": 0, "mode": mode,
    }
    if active_cus is not None:
        row["active_cus"] = active_cus
    return row


def write_csv(path, rows):
    fields = (["active_cus"] if rows and "active_cus" in rows[0] else []) + CSV_FIELDS
    with open(path, "w", newline="") as f:
        writer = csv.DictWriter(f, fieldnames=fields)
        writer.writeheader()
        writer.writerows(rows)


def bench_matmul(input_yaml, init_type="randn", shuffle=False, output_csv=None, write_csv_freq=100, verbose=False, **kw):
    import yaml
    with open(input_yaml) as f:
        cases = list(yaml.safe_load(f))
    if shuffle:
        random.shuffle(cases)
    rows = []
    for i, case in enumerate(cases):
        row = bench_case(case, init_type, **kw)
        rows.append(row)
        if verbose:
            print(f"m={row['m']} n={row['n']} k={row['k']} {row['in_dtype']}->{row['out_dtype']} "
                  f"{row['transA']}{row['transB']} mode={row['mode']} tile={row['macro_tile']} "
                  f"{row['tritonblas_gflops'] / 1e3:.1f} TFLOP/s {row['us']:.1f} us", flush=True)
        if output_csv and (i % write_csv_freq == 0 or i + 1 == len(cases)):
            write_csv(output_csv, rows)
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--input-yaml", required=True)
    ap.add_argument("--output-csv")
    ap.add_argument("--init_type", default="randn", choices=["hpl", "trig_float", "zeros", "randn"])
    ap.add_argument("--shuffle-bench", action="store_true")
    ap.add_argument("--csv-write-freq", type=int, default=100)
    ap.add_argument("--print-verbose", action="store_true")
    ap.add_argument("--enable-streamk", action="store_true")
    ap.add_argument("--work-stealing", action="store_true")
    ap.add_argument("--checkcorrectness", action="store_true")
    ap.add_argument("--active-cus", type=int, default=None, help="restrict the launch grid to this many SMs")
    ap.add_argument("--cu-sweep", default=None, help="comma-separated SM counts; one pass over the YAML per count")
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeat", type=int, default=100)
    args = ap.parse_args(argv)
    common = dict(init_type=args.init_type, shuffle=args.shuffle_bench, write_csv_freq=args.csv_write_freq,
                  verbose=args.print_verbose, enable_streamk=args.enable_streamk, work_stealing=args.work_stealing,
                  check=args.checkcorrectness, n_warmup=args.warmup, n_repeat=args.repeat)
    if args.cu_sweep:
        rows = []
        for count in (int(x) for x in args.cu_sweep.split(",")):
            rows += bench_matmul(args.input_yaml, active_cus=count, **common)
            if args.output_csv:
                write_csv(args.output_csv, rows)
    else:
        rows = bench_matmul(args.input_yaml, output_csv=args.output_csv, active_cus=args.active_cus, **common)
    if args.output_csv:
        print(f"{len(rows)} rows written to {args.output_csv}")
    return rows


if __name__ == "__main__":
    main()
