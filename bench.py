"""Headline benchmark: bf16 GEMM 8192^3 (TN layout) on B200, through tritonblas_b200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: `--gemms-per-step` GEMMs of the workload's
shape. Prints ONE JSON line (rank 0). Keys:
  value      whole-job TFLOP/s with operands resident in HBM, CUDA-event timed, max over ranks
  e2e        the same metric through the public API with HOST (pinned) operands: H2D of A and B and D2H of C inside the
             timed region, every step
  roofline   the dominant kernel against the measured cuBLAS bf16 throughput (MEASURED_PEAKS.json) or HBM bandwidth
  cpu_baseline   the reference semantics (fp32-accumulate torch.matmul) on the host cores, on a bounded row sample
With --gpus N > 1 (launched under torchrun) the 8192^3 product is N-sharded: rank r computes C[:, r*N/P:(r+1)*N/P] with
the full A and its column block of B, then the ranks all-gather C over NCCL (total work fixed: "strong" scaling).
--impl reference times the reference's CPU implementation of the path (torch.matmul semantics) instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, N, K, dtype, streamk, bound)
    "bf16_8192": (8192, 8192, 8192, "bf16", False, "tensor"),
    "bf16_skinny_m1": (1, 28672, 8192, "bf16", True, "hbm"),
    "bf16_skinny_m16": (16, 28672, 8192, "bf16", True, "hbm"),
    "bf16_skinny_m128": (128, 28672, 8192, "bf16", True, "hbm"),
    "fp16_1024": (1024, 1024, 1024, "fp16", False, "tensor"),
}
DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        for p in self.samples:
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_tflops(M, N, K, dtype, target_seconds, seed=0):
    """Reference semantics on the host: torch.matmul of the fp32 up-cast operands, cast to the output type
    (the contract of include/tritonblas/kernels/stages/matrix_view.py:263-301). Timed on a bounded sample of rows."""
    from oracle import gemm_oracle
    g = torch.Generator().manual_seed(seed)
    b = (torch.randn(K, N, generator=g) * 0.02).to(dtype)
    rows = min(M, 64)
    a = (torch.randn(rows, K, generator=g) * 0.02).to(dtype)
    t0 = time.perf_counter()
    gemm_oracle.gemm_ref(a, b, dtype)
    dt = time.perf_counter() - t0
    # grow the sample toward the time budget (the first call also pays the fp32 conversion of B)
    rows2 = int(min(M, max(rows, rows * target_seconds / max(dt, 1e-3) * 0.5)))
    rows2 = max(rows2 - rows2 % 64, min(M, 64))
    a = (torch.randn(rows2, K, generator=g) * 0.02).to(dtype)
    t0 = time.perf_counter()
    gemm_oracle.gemm_ref(a, b, dtype)
    dt = time.perf_counter() - t0
    return 2.0 * rows2 * N * K / dt / 1e12, rows2, dt


def run_reference(args, M, N, K, dtype, rank, world):
    if rank != 0:
        return
    times, rows = [], 0
    for i in range(args.warmup + args.steps):
        tf, rows, dt = cpu_reference_tflops(M, N, K, dtype, target_seconds=max(2.0, 20.0 / max(args.steps, 1)), seed=i)
        if i >= args.warmup:
            times.append((tf, dt))
    tf = sum(t[0] for t in times) / len(times)
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(t[1] for t in times) / len(times),
        "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
        "dtype": args.dtype_name, "data": "synthetic",
        "config": {"workload": f"{args.workload}: {args.dtype_name} GEMM M={M} N={N} K={K}, reference semantics "
                               f"(fp32-accumulate torch.matmul) on host cores"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{rows} of {M} rows of A per step against the full B"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--gemms-per-step", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-operand leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    M, N, K, dtype_name, streamk, bound = WORKLOADS[args.workload]
    dtype = DTYPES[dtype_name]
    args.dtype_name = dtype_name

    if args.impl == "reference":
        run_reference(args, M, N, K, dtype, rank, world)
        return

    import tritonblas_b200 as tb
    from tritonblas_b200 import _lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    # ---- synthetic operands (seeded; values ~ N(0,1)*0.02 as the configuration states). TN layout: both K-contiguous.
    n_local = N // world
    g = torch.Generator().manual_seed(1234)
    nsets = 2  # rotate operand sets so consecutive GEMMs never reuse the same operands
    A_host = [(torch.randn(M, K, generator=g) * 0.02).to(dtype).pin_memory() for _ in range(nsets)]
    B_host = [(torch.randn(n_local, K, generator=torch.Generator().manual_seed(99 + rank + 7 * i)) * 0.02).to(dtype).pin_memory()
              for i in range(nsets)]
    A = [t.to(dev, non_blocking=True) for t in A_host]
    Bt = [t.to(dev, non_blocking=True) for t in B_host]     # (N_local, K) row-major
    C = [torch.empty(M, n_local, dtype=dtype, device=dev) for _ in range(nsets)]
    C_host = torch.empty(M, n_local, dtype=dtype).pin_memory()
    Cg = torch.empty(world, M, n_local, dtype=dtype, device=dev) if world > 1 else None
    sel = tb.OrigamiMatmulSelector(M, n_local, K, dtype, dtype, dtype, dev, streamk=streamk)
    cfg = tb.matmul_preamble(sel)
    gps = args.gemms_per_step
    flops_step = 2.0 * M * N * K * gps          # whole job (all ranks)
    stream = torch.cuda.current_stream()

    def step(i, events=None):
        for j in range(gps):
            s = (i * gps + j) % nsets
            if events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            tb.matmul_lt(A[s], Bt[s].T, C[s], sel, cfg, enable_streamk=streamk)
            if events is not None:
                e1.record(stream)
                events.append((e0, e1))
            if world > 1:
                dist.all_gather_into_tensor(Cg, C[s])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    launches0 = _lib.lib.tb_launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    kernel_events = []
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record(stream)
    for i in range(args.steps):
        step(i, kernel_events)
    t_end.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = _lib.lib.tb_launch_count() - launches0
    ms_total = t_start.elapsed_time(t_end)
    kernel_ms = sum(e0.elapsed_time(e1) for e0, e1 in kernel_events) / max(len(kernel_events), 1)
    status = tb.device_status(local_rank)

    # ---- end to end through the public API with host operands (H2D of A and B, D2H of C inside the timed region)
    def e2e_step(i):
        s = i % nsets
        a = A_host[s].to(dev, non_blocking=True)
        b = B_host[s].to(dev, non_blocking=True)
        c = tb.matmul(a, b.T, enable_streamk=streamk)
        if world > 1:
            dist.all_gather_into_tensor(Cg, c)
        C_host.copy_(c, non_blocking=True)

    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    for i in range(2 if e2e_steps else 0):
        e2e_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(e2e_steps):
        e2e_step(i)
    e1.record(stream)
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 1e-6)

    if world > 1:
        t = torch.tensor([ms_total, e2e_ms, kernel_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, e2e_ms, kernel_ms = t.tolist()
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt.item())

    if rank == 0:
        peaks = measured_peaks()
        esize = 2
        value = flops_step * args.steps / (ms_total * 1e-3) / 1e12
        e2e_value = 2.0 * M * N * K * e2e_steps / (e2e_ms * 1e-3) / 1e12
        if bound == "tensor":
            timed_s = ms_total * 1e-3
            peak = peaks["bf16_tflops"] if timed_s < 1.0 else peaks["bf16_tflops_sustained"]
            peak_kind = ("burst" if timed_s < 1.0 else "sustained") + f" cuBLAS bf16, {peaks['source']}"
            achieved = 2.0 * M * n_local * K / (kernel_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "peak_kind": peak_kind, "kernel_ms": kernel_ms,
                    "frac_of_nominal_dense": achieved / 2250.0}
        else:
            alg_bytes = esize * (M * K + K * n_local + M * n_local)
            achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None, "peak_kind": f"copy, {peaks['source']}",
                    "kernel_ms": kernel_ms}
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
            "config": {"workload": f"{args.workload}: {dtype_name} GEMM M={M} N={N} K={K} TN layout, fp32 accumulate, "
                                   f"{dtype_name} out, inputs N(0,1)*0.02" + (", stream-K" if streamk else ""),
                       "gemms_per_step": gps, "tile": f"{sel.block_m}x{sel.block_n}x{sel.block_k}",
                       "cta_pair": sel.cta_pair, "l2_policy": "operand sets rotate; each set (A+B+C) exceeds L2",
                       "parallelism": f"N-sharded x{world} + all-gather of C" if world > 1 else "single GPU"},
            "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": esize * (M * K + n_local * K), "d2h_bytes_per_step": esize * M * n_local,
                    "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks, "device_status": status,
        }
        if not args.no_cpu_baseline and world == 1:
            tf, rows, dt = cpu_reference_tflops(M, N, K, dtype, target_seconds=15.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"{rows} of {M} rows of A against the full B, {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
