"""Headline benchmark of the GEMM hot path on B200, through tritonblas_b200's public API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload: bf16 GEMM 8192^3, TN layout, inputs N(0,1)*0.02 (the configuration the headline metric is quoted on).
One "step" is one pass of the hot path over one batch of synthetic input (`--gemms-per-step` products of that shape).
Prints ONE JSON line (rank 0):
  value        whole-job TFLOP/s with operands resident in HBM, CUDA-event timed, max over ranks
  e2e          the same metric through the public API with HOST (pinned) operands: H2D of the inputs and D2H of the result
               inside the timed region, every step
  roofline     the dominant kernel against the measured cuBLAS bf16 throughput / HBM copy bandwidth (MEASURED_PEAKS.json)
  parity_check a fixed sample of the result of one more step, on every rank, against the CPU oracle (outside the timed
               region): rows x columns of C including columns every other rank computed
  cpu_baseline the reference semantics (fp32-accumulate torch.matmul) on the host cores, on a bounded sample
With the default workload the line also carries (each measured after the headline, outside `value`):
  moe / moe_nccl  the expert-parallel MoE step (64 experts, top-8 of 16384 tokens, hidden 4096, ffn 1536, Zipf routing) at
               this GPU count: whole-job TFLOP/s, ms per step, rows per rank, its own parity_check. On several GPUs `moe`
               exchanges tokens through peer-mapped memory, `moe_nccl` through NCCL all-to-all.
  cublas_same_run, sustained, workloads   (1 GPU) torch.matmul on the same operands in the same run; a >= 1.5 s
               back-to-back block with clocks; kernel-level roofline lines of the FP8, MXFP4, quantiser and decode shapes.
With --gpus N > 1 (under torchrun) the default workload is N-sharded: rank r computes C[:, r*N/P:(r+1)*N/P] from the full A
and its column block of B and the GEMM epilogue pushes every tile into all ranks' gathered C over NVLink (total work
fixed: "strong" scaling); `--nccl-gather` gathers with NCCL instead. `--workload moe` runs only the MoE step.
`--impl reference` times the reference's CPU implementation of the path (its matmul semantics via torch.matmul).
"""
import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

# A rank of a multi-GPU run must never be bound to an NVLink multicast object (a rank that dies while bound raises
# faults on its peers); this library only uses ordinary peer loads and stores.
os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FP8 = torch.float8_e4m3fn
NOMINAL_TFLOPS = {"bf16": 2250.0, "fp16": 2250.0, "fp8": 4500.0, "mxfp4": 9000.0}

# name: dict(M, N, K, dtype, streamk, bound[, static_b]). static_b: the decode shapes promise the library that B (the
# weights) is not written by anything in flight, which lets a kernel start fetching it while its predecessor drains.
WORKLOADS = {
    "bf16_8192": dict(M=8192, N=8192, K=8192, dtype="bf16", streamk=False, bound="tensor"),
    "fp16_1024": dict(M=1024, N=1024, K=1024, dtype="fp16", streamk=False, bound="tensor"),
    "bf16_skinny_m1": dict(M=1, N=28672, K=8192, dtype="bf16", streamk=True, bound="hbm", static_b=True),
    "bf16_skinny_m16": dict(M=16, N=28672, K=8192, dtype="bf16", streamk=True, bound="hbm", static_b=True),
    "bf16_skinny_m128": dict(M=128, N=28672, K=8192, dtype="bf16", streamk=True, bound="hbm", static_b=True),
    "fp8_m16": dict(M=16, N=28672, K=8192, dtype="fp8", streamk=True, bound="hbm", static_b=True),
    "fp8_m256": dict(M=256, N=28672, K=8192, dtype="fp8", streamk=False, bound="hbm"),
    "fp8_m4096": dict(M=4096, N=28672, K=8192, dtype="fp8", streamk=False, bound="tensor"),
    "mxfp4_8192": dict(M=8192, N=8192, K=8192, dtype="mxfp4", streamk=False, bound="tensor"),
    "mxfp4_quant": dict(M=8192, N=8192, K=8192, dtype="mxfp4", streamk=False, bound="hbm"),
    "moe": dict(M=16384 * 8, N=0, K=0, dtype="bf16", streamk=False, bound="tensor"),
}
# kernel-level lines added to the default 1-GPU run
EXTRA_WORKLOADS = ["fp8_m4096", "mxfp4_8192", "mxfp4_quant", "bf16_skinny_m16", "bf16_skinny_m128", "fp8_m16"]
TORCH_DTYPES = {"bf16": torch.bfloat16, "fp16": torch.float16}
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the workload's dominant kernel, from the ncu captures
# summarised under profiles/ (same shapes; a capture is not repeated inside the bench)
NCU_TRAFFIC_BYTES = {"bf16_8192": 0.794e9 + 0.124e9, "mxfp4_8192": 0.1565e9 + 0.1132e9, "mxfp4_quant": 0.1343e9 + 0.0078e9,
                     "bf16_skinny_m16": 0.4718e9 + 0.0075e9, "fp8_m4096": 0.5615e9 + 0.2225e9}
MOE = dict(experts=64, topk=8, tokens=16384, hidden=4096, ffn=1536)


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
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)  # let the first samples arrive before the timed region starts
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append((time.time(), parts))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [p for t, p in self.samples if t_begin <= t <= t_end + 0.06] or [p for _, p in self.samples[-3:]]
        sm, reasons, mx, power = [], set(), None, []
        for p in inside:
            try:
                sm.append(float(p[0]))
                mx = float(p[1])
                power.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


# ------------------------------------------------------------------------------------------ CPU reference leg
def cpu_reference_tflops(M, N, K, dtype, target_seconds, seed=0):
    """Reference semantics on the host: torch.matmul of the fp32 up-cast operands, one cast to the output type
    (include/tritonblas/kernels/stages/matrix_view.py:263-301). Timed on a bounded sample of A's rows."""
    from oracle import gemm_oracle
    g = torch.Generator().manual_seed(seed)
    b = (torch.randn(K, N, generator=g) * 0.02).to(dtype)
    rows = min(M, 64)
    a = (torch.randn(rows, K, generator=g) * 0.02).to(dtype)
    t0 = time.perf_counter()
    gemm_oracle.gemm_ref(a, b, dtype)
    dt = time.perf_counter() - t0
    rows2 = int(min(M, max(rows, rows * target_seconds / max(dt, 1e-3) * 0.5)))
    rows2 = max(rows2 - rows2 % 64, min(M, 64))
    a = (torch.randn(rows2, K, generator=g) * 0.02).to(dtype)
    # repeat the sample until about target_seconds of CPU work have been timed (a fast host finishes one pass early)
    reps, total = 0, 0.0
    while reps == 0 or (total < 0.7 * target_seconds and reps < 64):
        t0 = time.perf_counter()
        gemm_oracle.gemm_ref(a, b, dtype)
        total += time.perf_counter() - t0
        reps += 1
    dt = total / reps
    return 2.0 * rows2 * N * K / dt / 1e12, rows2, total


def dense_label(wl):
    M, N, K = wl["M"], wl["N"], wl["K"]
    fp8 = wl["dtype"] == "fp8"
    return (f"{wl['dtype']} GEMM M={M} N={N} K={K} TN layout, fp32 accumulate, "
            f"{'bf16' if fp8 else wl['dtype']} out, inputs N(0,1)*0.02"
            + (", per-token x per-channel e4m3 scales in the epilogue" if fp8 else "")
            + (", stream-K" if wl["streamk"] else ""))


def run_reference(args, wl, rank):
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)   # torchrun pins OMP_NUM_THREADS=1; the CPU arm uses every host core
    if args.workload == "moe":
        M, N, K = 2048, MOE["hidden"], MOE["ffn"] * 2   # one average expert's gate/up projection as the sample shape
    else:
        M, N, K = wl["M"], wl["N"], wl["K"]
    dtype = TORCH_DTYPES.get(wl["dtype"], torch.bfloat16)   # fp8 / fp4 codes are up-cast to fp32 by the reference check
    samples = []
    for i in range(args.warmup + args.steps):
        tf, rows, dt = cpu_reference_tflops(M, N, K, dtype, target_seconds=max(1.0, 20.0 / max(args.steps, 1)), seed=i)
        if i >= args.warmup:
            samples.append((tf, 2.0 * rows * N * K / tf / 1e12, rows))
    tf = sum(s[0] for s in samples) / len(samples)
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(s[1] for s in samples) / len(samples),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        # the same workload as the other arm (same name and description); how this arm runs it is said under "arm"
        "config": {"workload": f"{args.workload}: " + (dense_label(wl) if args.workload != "moe" and wl["dtype"] != "mxfp4"
                                                        else f"GEMM M={M} N={N} K={K}"),
                   "gemms_per_step": args.gemms_per_step if args.workload != "moe" else 1,
                   "arm": "reference semantics (fp32-accumulate torch.matmul, one cast) on the host cores, bounded row sample"},
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{samples[-1][2]} of {M} rows of A per step against the full B"},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _parity(got, ref, rtol):
    """(ok, max error relative to rtol * (|ref| + rms)) of a sample against the oracle's fp32 values."""
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    rms = max(ref.pow(2).mean().sqrt().item(), 1e-30)
    err = (got - ref).abs()
    ok = bool(torch.isfinite(got).all()) and bool((err <= rtol * ref.abs() + rtol * rms).all())
    return ok, float(err.max().item()), rms


def _b_shard_host(rank, set_index, n_local, K):
    """Rank `rank`'s block of B for operand set `set_index` (bf16, (n_local, K)): every rank can rebuild any block."""
    g = torch.Generator().manual_seed(99 + rank + 7 * set_index)
    return (torch.randn(n_local, K, generator=g) * 0.02).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------ workloads (our arm)
class DenseWorkload:
    """bf16 / fp16 / fp8 GEMM, optionally N-sharded over the ranks with an all-gather of C."""

    def __init__(self, args, wl, dev, rank, world):
        import tritonblas_b200 as tb
        from tritonblas_b200 import utils
        self.tb, self.wl, self.dev, self.world, self.rank = tb, wl, dev, world, rank
        M, N, K = wl["M"], wl["N"], wl["K"]
        self.M, self.K = M, K
        self.n_local = N // world
        self.N = N
        self.fp8 = wl["dtype"] == "fp8"
        self.out_dtype = torch.bfloat16 if self.fp8 else TORCH_DTYPES[wl["dtype"]]
        self.in_dtype = FP8 if self.fp8 else self.out_dtype
        self.streamk = wl["streamk"]
        self.static_b = bool(wl.get("static_b", False))
        nsets = 2 if M * K + self.n_local * K < (1 << 29) else 1
        # small operands: rotate enough sets to exceed the 126 MB L2
        set_bytes = (M * K + self.n_local * K) * (1 if self.fp8 else 2) + M * self.n_local * 2
        while nsets * set_bytes < (160 << 20) and nsets < 64:
            nsets += 1
        self.nsets = nsets
        g = torch.Generator().manual_seed(1234)
        self.A_host, self.B_host, self.a_s, self.b_s = [], [], [], []
        for i in range(nsets):
            a = (torch.randn(M, K, generator=g) * (1.0 if self.fp8 else 0.02)).to(torch.bfloat16)
            b = _b_shard_host(rank, i, self.n_local, K)
            if self.fp8:
                a8, a_s = utils.quantize_tensor_per_channel(a, FP8, axis=1)
                b8, b_s = utils.quantize_tensor_per_channel(b, FP8, axis=1)   # rows of (N, K) = output channels
                a, b = a8, b8
                self.a_s.append(a_s.to(dev))
                self.b_s.append(b_s.to(dev))
            else:
                a, b = a.to(self.in_dtype), b.to(self.in_dtype)
            self.A_host.append(a.pin_memory())
            self.B_host.append(b.pin_memory())
        self.A = [t.to(dev) for t in self.A_host]
        self.Bt = [t.to(dev) for t in self.B_host]                       # (n_local, K): K-contiguous B
        self.C = [torch.empty(M, self.n_local, dtype=self.out_dtype, device=dev) for _ in range(min(nsets, 4))]
        self.C_host = torch.empty(M, self.n_local, dtype=self.out_dtype).pin_memory()
        self.Cg = torch.empty(world * M, self.n_local, dtype=self.out_dtype, device=dev) if world > 1 else None
        self.layers = None
        if world > 1 and not self.fp8 and not args.nccl_gather:
            # fused path: the GEMM epilogue pushes every tile into all ranks' gathered buffers (symmetric memory)
            from tritonblas_b200 import distributed as tbd
            self.layers = [tbd.ColumnShardedGemm(bt) for bt in self.Bt]
            for layer in self.layers:
                layer.enable_fused_gather(M, self.out_dtype, block_n=args.fused_block_n or None)
        self.gps = max(int(args.gemms_per_step), 1)
        self.overlap_tail = 0.0
        if self.layers is not None:
            # How the block reaches the peers. Measured (TFLOP/s of the whole job, bf16 8192^3):
            #   2 GPUs: pushes from the epilogue hide behind compute (2778); sending the last 15 % / 30 % of the tiles from a
            #           side stream instead: 2768 / 2712.
            #   4 GPUs: epilogue pushes 4059-4084 (they hold accumulators back while the link is busy, and the link idles
            #           during a launch's first wave); last 15 / 30 / 50 % from a side stream: 4028 / 3977 / 3801-3966; the
            #           epilogue pushes with only the closing barrier on a side stream: 4196-4236; the whole block by this
            #           library's copy kernel on a side stream beside the next product: 3350 (the copy kernel shares SMs
            #           with the GEMM: it runs at half its stand-alone rate and the GEMM a fifth slower; kept off the GEMM's
            #           SMs, with the GEMM on 8-16 fewer: 3191-3214); the whole block by asynchronous copies (copy
            #           engines) beside the next product: 4407-4441.
            #           The first tile groups from the epilogue and the rows of the last 25 / 50 / 75 % by copy engines:
            #           4202 / 4094 / 3977 against 4273 for the whole block by copy engines in the same call.
            #   8 GPUs: epilogue pushes 4147, with the closing barrier on a side stream 4300 (0.256 ms per product, 459 GB/s
            #           out of every GPU); the last half of the tiles by the copy kernel on a side stream instead: 4782 (a
            #           rank's shard is 128 tiles on 74 CTA pairs, which leaves the copy kernel room); the whole block by
            #           copy engines: 3204 (seven copies out and seven in per GPU); NCCL all-gather after the GEMM: 3400.
            auto = 1.0 if world == 4 else (0.5 if world >= 8 else 0.0)
            self.overlap_tail = auto if args.overlap_tail < 0 else float(args.overlap_tail)
        # --copy-engine 1: the whole block by copy engines when overlap_tail is 1; 2: also a partial tail (the rows of the
        # last tile groups by copy engines, the first groups from the epilogue) instead of the copy kernel
        self.copy_engine = (int(args.copy_engine) == 1 and self.overlap_tail >= 1.0) or (int(args.copy_engine) == 2 and self.overlap_tail > 0)
        self.side_barrier = self.layers is not None and self.overlap_tail <= 0 and bool(args.side_barrier)
        self.sel = tb.OrigamiMatmulSelector(M, self.n_local, K, self.in_dtype, self.in_dtype, self.out_dtype, dev,
                                            streamk=self.streamk)
        self.cfg = tb.matmul_preamble(self.sel)
        es = 1 if self.fp8 else 2
        self.flops = 2.0 * M * N * K
        self.kernel_flops = 2.0 * M * self.n_local * K
        self.kernel_bytes = es * (M * K + K * self.n_local) + 2 * M * self.n_local + (4 * (M + self.n_local) if self.fp8 else 0)
        self.h2d = es * (M * K + self.n_local * K)
        self.d2h = 2 * M * self.n_local
        self.label = dense_label(wl)
        if world == 1:
            how = "single GPU"
        elif self.layers is None:
            how = f"N-sharded x{world}, NCCL all-gather of C"
        elif self.overlap_tail <= 0:
            how = (f"N-sharded x{world}, epilogue pushes C tiles to all ranks over NVLink (symmetric memory) + barrier"
                   + (" on a side stream (the next product does not wait for it; the timed region does)" if self.side_barrier else ""))
        elif self.copy_engine and self.overlap_tail < 1.0:
            how = (f"N-sharded x{world}, the first tile groups of every product's C go to all ranks from the epilogue over NVLink, "
                   f"the rows of the last groups (about {self.overlap_tail:.2f} of the tiles) by asynchronous peer copies on side "
                   "streams beside the next product (symmetric memory) + barrier; the timed region ends after every transfer "
                   "and barrier")
        elif self.copy_engine:
            how = (f"N-sharded x{world}, every product's block of C is copied into all ranks' gathered buffers (symmetric "
                   "memory) by asynchronous peer copies on side streams beside the next product + barrier; the timed "
                   "region ends after every transfer and barrier")
        else:
            how = (f"N-sharded x{world}, the last {self.overlap_tail:.2f} of every product's C tiles are copied to all ranks over "
                   "NVLink by a kernel on a side stream beside the next product, the rest by the epilogue (symmetric memory) "
                   "+ barrier; the timed region ends after every transfer and barrier")
        self.extra = {"tile": f"{self.sel.block_m}x{self.sel.block_n}x{self.sel.block_k}", "cta_pair": self.sel.cta_pair,
                      "operand_sets": nsets, "parallelism": how}
        if self.static_b:
            self.extra["static_b"] = True
        # end-to-end leg: copies and compute on separate streams, double-buffered device operands
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.a_dev = [torch.empty_like(self.A[0]) for _ in range(2)]
        self.b_dev = [torch.empty_like(self.Bt[0]) for _ in range(2)]
        self.c_dev = [torch.empty(M, self.n_local, dtype=self.out_dtype, device=dev) for _ in range(2)]
        self.ev_in = [None, None]
        self.ev_c = [None, None]
        self.ev_out = [None, None]

    def gemm(self, i, a=None, b_t=None, c=None):
        s = i % self.nsets
        a = self.A[s] if a is None else a
        b_t = self.Bt[s] if b_t is None else b_t
        c = self.C[i % len(self.C)] if c is None else c
        static = self.static_b and b_t is self.Bt[s]   # only the resident weights; the end-to-end leg's are copied in
        if self.fp8:
            self.tb.matmul_a8w8_lt(a, b_t.T, self.a_s[s], self.b_s[s], c, self.sel, self.cfg, enable_streamk=self.streamk,
                                   static_b=static)
        else:
            self.tb.matmul_lt(a, b_t.T, c, self.sel, self.cfg, enable_streamk=self.streamk, static_b=static)
        return c

    def step(self, i, dist):
        if self.layers is not None:
            # two gathered buffers alternate, so the opening barrier is not needed (see forward_fused). With overlap_tail
            # the tiles of a product cross NVLink from a side stream while the next product computes (products are
            # independent: nothing reads a gathered result before `finish`); the launch loop never waits, the timed
            # region ends only after every product's transfer and closing barrier (`finish`).
            return self.layers[i % self.nsets].forward_fused(self.A[i % self.nsets], pre_barrier=self.nsets < 2,
                                                             overlap_tail=self.overlap_tail,
                                                             tail_by_copy_engine=self.copy_engine,
                                                             barrier_on_side_stream=self.side_barrier)
        c = self.gemm(i)
        if self.world > 1:
            dist.all_gather_into_tensor(self.Cg, c)
            return self.Cg.view(self.world, self.M, self.n_local)
        return c

    def finish(self):
        """Make the launching stream wait for everything the steps left on side streams (inside the timed region)."""
        if self.layers is not None and (self.overlap_tail > 0 or self.side_barrier):
            for layer in self.layers:
                layer.wait_gathered()

    def cublas_step(self, i):
        """torch.matmul (cuBLAS), or torch._scaled_mm (cuBLASLt, row-wise scales) for fp8, on the same operands, for the
        same-run comparison; not part of `value`."""
        s = i % self.nsets
        if self.fp8:
            torch._scaled_mm(self.A[s], self.Bt[s].T, scale_a=self.a_s[s].view(-1, 1), scale_b=self.b_s[s].view(1, -1),
                             out_dtype=torch.bfloat16, out=self.C[i % len(self.C)])
        else:
            torch.matmul(self.A[s], self.Bt[s].T, out=self.C[i % len(self.C)])

    def e2e_step(self, i, dist):
        """Host operands in, host result out, through the public API. H2D of step i+1 and D2H of step i-1 run on their own
        streams beside the GEMM of step i; every step still copies its own inputs and its own result."""
        s, j = i % self.nsets, i % 2
        main = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            if self.ev_c[j] is not None:
                self.s_in.wait_event(self.ev_c[j])          # the GEMM that last read these device operands is done
            self.a_dev[j].copy_(self.A_host[s], non_blocking=True)
            self.b_dev[j].copy_(self.B_host[s], non_blocking=True)
            self.ev_in[j] = self.s_in.record_event()
        main.wait_event(self.ev_in[j])
        if self.ev_out[j] is not None:
            main.wait_event(self.ev_out[j])                 # the previous result in this buffer has left for the host
        c = self.c_dev[j]
        if self.layers is not None:
            # the same fused path as `value`: this rank's block goes to every rank's gathered buffer from the epilogue
            gathered = self.layers[j].forward_fused(self.a_dev[j], pre_barrier=self.nsets < 2, b_shard_t=self.b_dev[j])
            c = gathered[self.rank]
        elif self.fp8:
            self.tb.matmul_a8w8(self.a_dev[j], self.b_dev[j].T, self.a_s[s], self.b_s[s], c, enable_streamk=self.streamk)
        else:
            self.tb.matmul(self.a_dev[j], self.b_dev[j].T, out=c, enable_streamk=self.streamk)
        if self.world > 1 and self.layers is None:
            dist.all_gather_into_tensor(self.Cg, c)
        self.ev_c[j] = main.record_event()
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_c[j])
            self.C_host.copy_(c, non_blocking=True)
            self.ev_out[j] = self.s_out.record_event()

    def e2e_finish(self):
        main = torch.cuda.current_stream()
        for ev in self.ev_out:
            if ev is not None:
                main.wait_event(ev)

    def parity_check(self, dist):
        """One more step on operand set 0; 64 rows x 256 columns of the (gathered) C, the columns spread evenly over
        every rank's block, against the CPU oracle."""
        from oracle import gemm_oracle
        out = self.step(0, dist)
        torch.cuda.synchronize()            # every stream of the device, the side stream of the tail copies included
        if dist is not None:
            dist.barrier()
        g = torch.Generator().manual_seed(2024)
        rows = torch.unique(torch.cat([torch.randint(0, self.M, (60,), generator=g),
                                       torch.tensor([0, min(127, self.M - 1), min(128, self.M - 1), self.M - 1])]))
        per = max(256 // self.world, 8)
        ok, worst = True, 0.0
        for r in range(self.world):
            cols = torch.unique(torch.cat([torch.randint(0, self.n_local, (per - 2,), generator=g),
                                           torch.tensor([0, self.n_local - 1])]))
            block = out[r] if self.world > 1 else out
            got = block[rows.to(self.dev)][:, cols.to(self.dev)]
            if self.fp8:      # single GPU only: the quantised operands and their scales are at hand
                ref = gemm_oracle.gemm_ref_f32(self.A[0][rows.to(self.dev)], self.Bt[0][cols.to(self.dev)].T,
                                               self.a_s[0][rows.to(self.dev)], self.b_s[0][cols.to(self.dev)])
            else:
                b_blk = _b_shard_host(r, 0, self.n_local, self.K).to(self.in_dtype)
                ref = gemm_oracle.gemm_ref_f32(self.A_host[0][rows], b_blk[cols].T)
            k, e, _ = _parity(got, ref, 1e-2)
            ok, worst = ok and k, max(worst, e)
        return ok, worst


class Mxfp4Workload:
    """MXFP4 GEMM 8192^3 (activations through the fused Hadamard+quantise kernel) or the quantise kernel alone."""

    def __init__(self, args, wl, dev, rank, world, quant_only):
        import tritonblas_b200 as tb
        from tritonblas_b200 import utils
        self.tb, self.utils, self.dev, self.quant_only = tb, utils, dev, quant_only
        M, N, K = wl["M"], wl["N"], wl["K"]
        self.M, self.N, self.K = M, N, K
        g = torch.Generator().manual_seed(4321)
        self.nsets = 2
        self.X_host = [torch.randn(M, K, generator=g).to(torch.bfloat16).pin_memory() for _ in range(self.nsets)]
        self.X = [t.to(dev) for t in self.X_host]
        w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(dev)
        self.qb, self.sb = utils.hadamard_mxfp4_quant(w, scale_atoms=True)       # weights: rotated and quantised offline
        del w
        self.q = [utils.hadamard_mxfp4_quant(x, scale_atoms=True) for x in self.X]
        self.C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        self.C_host = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()
        self.q_host = torch.empty(M, K // 2, dtype=torch.uint8).pin_memory()
        self.flops = self.kernel_flops = 2.0 * M * N * K
        if quant_only:
            self.kernel_bytes = M * K * 2 + M * K // 2 + M * K // 32
            self.label = f"fused 32-point Hadamard + MXFP4 quantise of a bf16 {M}x{K} activation (N(0,1))"
        else:
            self.kernel_bytes = (M * K + N * K) // 2 + (M * K + N * K) // 32 + 2 * M * N
            self.label = (f"MXFP4 GEMM M={M} N={N} K={K}: e2m1 operands, e8m0 scale per 32 K elements, bf16 out; sources "
                          f"bf16 N(0,1); activations pre-quantised by the fused Hadamard+quantise kernel (timed apart in e2e)")
        self.h2d, self.d2h = M * K * 2, (M * K // 2 + M * K // 32 if quant_only else 2 * M * N)
        self.extra = {"parallelism": "single GPU"}
        self.qout = utils.hadamard_mxfp4_quant(self.X[0], scale_atoms=True) if quant_only else None

    def step(self, i, dist):
        s = i % self.nsets
        if self.quant_only:
            return self.utils.hadamard_mxfp4_quant(self.X[s], scale_atoms=True, out=self.qout)
        return self.tb.matmul_fp4(self.q[s][0], self.qb, self.C, self.q[s][1], self.sb)

    def e2e_step(self, i, dist):
        x = self.X_host[i % self.nsets].to(self.dev, non_blocking=True)
        qa, sa = self.utils.hadamard_mxfp4_quant(x, scale_atoms=True)
        if self.quant_only:
            self.q_host.copy_(qa, non_blocking=True)
            return
        self.tb.matmul_fp4(qa, self.qb, self.C, sa, self.sb)
        self.C_host.copy_(self.C, non_blocking=True)

    def parity_check(self, dist):
        """Sampled rows: quantiser codes and scales bit-exact against the oracle; GEMM rows against the dequantised fp32
        product (rtol 1e-2 + 1e-2 rms)."""
        import numpy as np
        from oracle import mxfp4_oracle
        rows = [0, 1, 127, 128, 4095, self.M - 1] + torch.randint(0, self.M, (26,), generator=torch.Generator().manual_seed(3)).tolist()
        idx = torch.tensor(rows, device=self.dev)
        if self.quant_only:
            qa, sa = self.utils.hadamard_mxfp4_quant(self.X[0][idx].contiguous())
            ra = mxfp4_oracle.hadamard_quantize_mxfp4(self.X[0][idx].float().cpu().numpy())
            ok = bool(np.array_equal(qa.cpu().numpy(), ra[0]) and np.array_equal(sa.cpu().numpy(), ra[1]))
            return ok, 0.0 if ok else 1.0
        qa, sa = self.utils.hadamard_mxfp4_quant(self.X[0][idx].contiguous())
        qb, sb = self.utils.hadamard_mxfp4_quant(self._weights_again())
        c = torch.empty(len(rows), self.N, dtype=torch.bfloat16, device=self.dev)
        self.tb.matmul_fp4(qa, qb, c, sa, sb)
        ref = mxfp4_oracle.mxfp4_gemm_ref(qa.cpu().numpy(), sa.cpu().numpy(), qb.cpu().numpy(), sb.cpu().numpy())
        ok, e, _ = _parity(c, torch.from_numpy(np.asarray(ref, dtype=np.float32)), 1e-2)
        # and the timed launch's own output on the same rows (full-size operands, scale atoms from the quantiser)
        self.step(0, dist)
        ok2, e2, _ = _parity(self.C[idx], torch.from_numpy(np.asarray(ref, dtype=np.float32)), 1e-2)
        return ok and ok2, max(e, e2)

    def _weights_again(self):
        g = torch.Generator().manual_seed(4321)
        for _ in range(self.nsets):
            torch.randn(self.M, self.K, generator=g)
        return torch.randn(self.N, self.K, generator=g).to(torch.bfloat16).to(self.dev)


def _expert_weights(e, H, F, dev):
    """Expert e's [gate | up] (2F, H) and down (H, F) projections, bf16 N(0, 0.02): any rank can rebuild any expert."""
    g = torch.Generator(device=dev).manual_seed(5000 + e)
    w1 = (torch.randn(2 * F, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(H, F, generator=g, device=dev) * 0.02).to(torch.bfloat16)
    return w1, w2


class MoeWorkload:
    """Expert-parallel MoE projections: 64 experts, top-8 of 16384 tokens, hidden 4096, ffn 1536, Zipf(1.1) routing."""

    def __init__(self, args, wl, dev, rank, world, nccl=False):
        import tritonblas_b200 as tb
        from tritonblas_b200 import distributed as tbd
        self.tb, self.tbd, self.dev, self.world, self.rank = tb, tbd, dev, world, rank
        E, topk, T, H, F = MOE["experts"], MOE["topk"], MOE["tokens"], MOE["hidden"], MOE["ffn"]
        self.t_local = T // world
        epr = E // world
        g = torch.Generator().manual_seed(77)                       # same routing table on every rank
        p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.1
        p = (p / p.sum())[torch.randperm(E, generator=g)]
        ids_all = torch.multinomial(p.expand(T, E), topk, replacement=False, generator=g)
        self.ids_host = ids_all[rank * self.t_local:(rank + 1) * self.t_local].contiguous().pin_memory()
        gw = torch.Generator().manual_seed(78 + rank)
        self.wts = (torch.rand(self.t_local, topk, generator=gw) * 0.2 + 0.025).to(dev)   # routing weights, fp32
        gl = torch.Generator().manual_seed(1000 + rank)
        self.x_host = torch.randn(self.t_local, H, generator=gl).to(torch.bfloat16).pin_memory()
        self.x, self.ids = self.x_host.to(dev), self.ids_host.to(dev)
        # Expert placement: balanced over the ranks by the per-expert load of the routing table (greedy, equal number of
        # experts per rank); with the contiguous layout one rank of eight holds twice the mean rows under this Zipf routing.
        load = torch.bincount(ids_all.flatten(), minlength=E)
        place = tbd.balanced_expert_placement(load, world) if (world > 1 and not args.contiguous_experts) else None
        layout = torch.arange(E) if place is None else torch.argsort(place.long())     # layout position -> expert id
        mine = [_expert_weights(int(e), H, F, dev) for e in layout[rank * epr:(rank + 1) * epr]]
        w1 = torch.stack([m[0] for m in mine])
        w2 = torch.stack([m[1] for m in mine])
        del mine
        if nccl:
            self.moe = tbd.ExpertParallelMoE(w1, w2, E, None, expert_place=None if place is None else place.to(dev))
        else:
            # device-side plan, one dispatch and one combine kernel; on several GPUs the rows travel over peer-mapped
            # memory (two barriers), on one GPU the same kernels run on local buffers
            self.moe = tbd.PeerMemoryMoE(w1, w2, E, capacity=T * topk, expert_place=place)
        self.path = "local" if world == 1 else ("nccl" if nccl else "peer")
        self.out_host = torch.empty(self.t_local, H, dtype=torch.bfloat16).pin_memory()
        rows = T * topk
        self.flops = 2.0 * rows * (H * 2 * F + F * H)
        self.kernel_flops = self.flops / world
        self.kernel_bytes = 0
        self.h2d, self.d2h = self.t_local * H * 2 + self.t_local * topk * 8, self.t_local * H * 2
        self.rows_per_rank = load[layout].reshape(world, epr).sum(1).tolist()
        self.placement = "contiguous" if place is None else "balanced by expert load (greedy, equal experts per rank)"
        self.label = (f"grouped MoE GEMM bf16: {E} experts, top-{topk} of {T} tokens, hidden {H}, ffn {F}, gate/up + down "
                      f"projections, Zipf(1.1) routing (seeded), SwiGLU between (fused into the gate/up epilogue, outside "
                      f"the FLOP count)")
        self.extra = {"parallelism": (f"expert-parallel x{world}, " + ("dispatch/combine kernels over NVLink peer memory"
                                      if self.path == "peer" else "NCCL all-to-all dispatch/combine")) if world > 1
                      else "single GPU", "rows_per_rank": self.rows_per_rank, "expert_placement": self.placement}

    def step(self, i, dist):
        return self.moe.forward(self.x, self.ids, self.wts)[0]

    def e2e_step(self, i, dist):
        x = self.x_host.to(self.dev, non_blocking=True)
        ids = self.ids_host.to(self.dev, non_blocking=True)
        out, _ = self.moe.forward(x, ids, self.wts)
        self.out_host.copy_(out, non_blocking=True)

    def parity_check(self, dist):
        """64 of this rank's tokens (their eight experts live on any rank) against the CPU oracle; rtol 2e-2 + 2e-2 rms
        (two chained bf16 GEMMs and a bf16 weighted sum)."""
        from oracle import moe_oracle
        out = self.step(0, dist)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        H, F = MOE["hidden"], MOE["ffn"]
        toks = torch.unique(torch.cat([torch.randint(0, self.t_local, (62,), generator=torch.Generator().manual_seed(9 + self.rank)),
                                       torch.tensor([0, self.t_local - 1])])).tolist()
        cache = {}

        def weights(e):
            if e not in cache:
                w1, w2 = _expert_weights(e, H, F, self.dev)
                cache[e] = (w1.cpu(), w2.cpu())
            return cache[e]

        ref = moe_oracle.moe_ffn_ref(self.x_host, self.ids_host, self.wts, lambda e: weights(e)[0], lambda e: weights(e)[1], toks)
        got = out[torch.tensor(toks, device=self.dev)].float().cpu()
        rms = ref.pow(2).mean().sqrt().item()
        err = (got - ref).abs()
        # chained bf16 GEMMs: 2e-2 relative plus one bf16 ulp of the largest value (an intermediate may round the other way)
        ok = bool(torch.isfinite(got).all()) and bool((err <= 2e-2 * ref.abs() + 2e-2 * rms + 2 ** -8 * ref.abs().max()).all())
        return ok, float(err.max().item())


def make_workload(name, args, dev, rank, world, **kw):
    wl = WORKLOADS[name]
    if name == "moe":
        return MoeWorkload(args, wl, dev, rank, world, **kw)
    if wl["dtype"] == "mxfp4":
        return Mxfp4Workload(args, wl, dev, rank, world, quant_only=(name == "mxfp4_quant"))
    return DenseWorkload(args, wl, dev, rank, world)


class Runner:
    """Timing of step functions with CUDA events on the launching stream, barrier + synchronize on both sides."""

    def __init__(self, dev, rank, world, local_rank, dist):
        self.dev, self.rank, self.world, self.local_rank, self.dist = dev, rank, world, local_rank, dist
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, *values):
        if self.world == 1:
            return list(values)
        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def all_ok(self, ok, err):
        if self.world == 1:
            return bool(ok), float(err)
        t = torch.tensor([0.0 if ok else 1.0, err], device=self.dev, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t[0].item() == 0.0, t[1].item()

    def timed(self, step, n_warm, n_timed, clocks=True, first=0, finish=None, per_call_events=True):
        """(total ms, mean ms of one call, clocks, launches of this library) of n_timed calls of step(i). ``finish`` runs
        after the last call and before the closing event (joins side streams: their work is inside the timed region).
        ``per_call_events=False`` records nothing between the calls (an event between two kernels keeps the second from
        being scheduled while the first drains); the mean is then the whole region's time over the number of calls."""
        from tritonblas_b200 import _lib
        it = first
        for _ in range(n_warm):
            step(it)
            it += 1
        if finish is not None:
            finish()
        self.barrier()
        launches0 = _lib.lib.tb_launch_count()
        sampler = ClockSampler(self.local_rank) if (clocks and self.rank == 0) else None
        if sampler:
            sampler.start()
        events = []
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        wall0 = time.time()
        t0.record(self.stream)
        for _ in range(n_timed):
            if per_call_events:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                step(it)
                e1.record(self.stream)
                events.append((e0, e1))
            else:
                step(it)
            it += 1
        if finish is not None:
            finish()
        t1.record(self.stream)
        self.barrier()
        wall1 = time.time()
        ck = sampler.stop(wall0, wall1) if sampler else None
        launches = _lib.lib.tb_launch_count() - launches0
        total = t0.elapsed_time(t1)
        unit = sum(a.elapsed_time(b) for a, b in events) / len(events) if events else total / n_timed
        if finish is not None:
            unit = total / n_timed      # calls overlap one another across streams: only the whole region's time counts
        total, unit = self.max_over_ranks(total, unit)
        if self.world > 1:
            lt = torch.tensor([launches], device=self.dev, dtype=torch.int64)
            self.dist.all_reduce(lt)
            launches = int(lt.item())
        return total, unit, ck, int(launches)


def roofline_of(name, w, unit_ms, timed_s, peaks, world):
    wl = WORKLOADS[name]
    if wl["bound"] == "tensor":
        achieved = w.kernel_flops / (unit_ms * 1e-3) / 1e12
        nominal = NOMINAL_TFLOPS[wl["dtype"]]
        if wl["dtype"] in ("bf16", "fp16"):
            peak = peaks["bf16_tflops"] if timed_s < 1.0 else peaks["bf16_tflops_sustained"]
            kind = ("burst" if timed_s < 1.0 else "sustained") + f" cuBLAS bf16 ({peaks['source']})"
        else:
            # no measured fp8 / fp4 tensor peak exists on this pool: the denominator is the nominal dense rate
            peak, kind = nominal, f"nominal dense {wl['dtype']} (no measured peak for this type)"
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(name) if world == 1 else None, "peak_kind": kind, "kernel_ms": unit_ms,
                "frac_of_nominal_dense": achieved / nominal}
    achieved = w.kernel_bytes / (unit_ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
            "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_kind": f"copy ({peaks['source']})", "kernel_ms": unit_ms,
            "algorithmic_bytes": w.kernel_bytes, "frac_of_nominal": achieved / 7700.0}


def release():
    gc.collect()
    torch.cuda.empty_cache()


def moe_block(args, run, nccl):
    """The MoE step at this GPU count: whole-job TFLOP/s (GEMM FLOPs of both projections / max-over-ranks time)."""
    w = MoeWorkload(args, WORKLOADS["moe"], run.dev, run.rank, run.world, nccl=nccl)
    n = max(5, min(args.steps, 12))
    total, unit, ck, launches = run.timed(lambda i: w.step(i, run.dist), 3, n, clocks=run.world == 1)
    ok, err = run.all_ok(*w.parity_check(run.dist))
    phases = None
    if w.path != "nccl":
        # one more step with an event after every phase (outside the timed steps): where the step's time goes on rank 0
        evs = []
        w.moe.forward(w.x, w.ids, w.wts, phase_events=evs)
        run.barrier()
        phases = {name: round(evs[i - 1][1].elapsed_time(ev), 4) for i, (name, ev) in enumerate(evs) if i > 0}
    out = {"value": w.flops * n / (total * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": total / n, "steps": n,
           "rows_per_rank": w.rows_per_rank, "expert_placement": w.placement, "path": w.path, "gpu_launches": launches,
           "parity_check": {"ok": ok, "max_err": err, "ranks_checked": run.world, "tokens_per_rank": 64,
                            "tolerance": "2e-2 * (|ref| + rms(ref)) + one bf16 ulp of max|ref| against the CPU oracle"},
           "frac_of_nominal_dense": w.flops * n / (total * 1e-3) / 1e12 / (NOMINAL_TFLOPS["bf16"] * run.world)}
    if ck:
        out["clocks"] = ck
    if phases is not None:
        out["phases_ms_rank0"] = phases
    del w
    release()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="bf16_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--gemms-per-step", type=int, default=4)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-operand leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true",
                    help="default workload: skip the MoE, sustained, cuBLAS and per-workload blocks (profiling runs)")
    ap.add_argument("--nccl-moe", action="store_true",
                    help="moe workload on several GPUs: NCCL all-to-all dispatch/combine instead of the peer-memory kernels")
    ap.add_argument("--fused-block-n", type=int, default=0,
                    help="multi-GPU default workload: tile width of the fused GEMM + push launch (0 = the library's choice)")
    ap.add_argument("--overlap-tail", type=float, default=-1.0,
                    help="multi-GPU default workload: share of every product's tiles pushed after the launch from a side "
                         "stream (0 = everything from the epilogue, -1 = chosen from the shard's compute and link times)")
    ap.add_argument("--side-barrier", type=int, default=1,
                    help="multi-GPU default workload with epilogue pushes: 1 = the closing barrier of every product runs on a "
                         "side stream (the next product does not wait for the other ranks), 0 = on the launching stream")
    ap.add_argument("--copy-engine", type=int, default=1,
                    help="with --overlap-tail 1: 1 = the block goes to the peers by asynchronous copies (copy engines), "
                         "0 = by this library's copy kernel")
    ap.add_argument("--contiguous-experts", action="store_true",
                    help="MoE on several GPUs: experts laid out over the ranks in id order instead of balanced by load")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="multi-GPU default workload: gather C with NCCL after the GEMM instead of the fused epilogue push")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, wl, rank)
        return

    import tritonblas_b200 as tb

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    run = Runner(dev, rank, world, local_rank, dist)
    default_line = args.workload == "bf16_8192" and not args.no_extras

    w = make_workload(args.workload, args, dev, rank, world, **({"nccl": args.nccl_moe} if args.workload == "moe" else {}))
    gps = 1 if args.workload == "moe" else args.gemms_per_step
    join = w.finish if (isinstance(w, DenseWorkload) and (w.overlap_tail > 0 or w.side_barrier)) else None
    ms_total, unit_ms, clocks, launches = run.timed(lambda i: w.step(i, dist), args.warmup * gps, args.steps * gps, finish=join)
    status = tb.device_status(local_rank)

    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 10))
    e2e_ms = 1e-6
    if e2e_steps:
        for i in range(2):
            w.e2e_step(i, dist)
        run.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(run.stream)
        for i in range(e2e_steps):
            w.e2e_step(i, dist)
        if hasattr(w, "e2e_finish"):
            w.e2e_finish()          # the last results' device-to-host copies are inside the timed region
        e1.record(run.stream)
        run.barrier()
        (e2e_ms,) = run.max_over_ranks(max(e0.elapsed_time(e1), 1e-6))

    p_ok, p_err = run.all_ok(*w.parity_check(dist))

    peaks = measured_peaks()
    line = None
    if rank == 0:
        value = w.flops * args.steps * gps / (ms_total * 1e-3) / 1e12
        e2e_value = w.flops * e2e_steps / (e2e_ms * 1e-3) / 1e12 if e2e_steps else 0.0
        roof = roofline_of(args.workload, w, unit_ms, ms_total * 1e-3, peaks, world)
        cfg = {"workload": f"{args.workload}: {w.label}", "gemms_per_step": gps,
               "l2_policy": "operand sets rotate; the rotated sets together exceed the 126 MB L2"}
        cfg.update(w.extra)
        line = {
            "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
            "config": cfg, "roofline": roof,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": w.h2d, "d2h_bytes_per_step": w.d2h,
                    "steps": e2e_steps,
                    "path": "fused epilogue push" if getattr(w, "layers", None) is not None else "public API"},
            "gpu_launches": int(launches), "clocks": clocks, "device_status": status,
        }
    parity = {"ok": p_ok, "max_err": p_err, "ranks_checked": world,
              "sample": "64 rows x 256 columns of the gathered C per rank, columns from every rank's block"
                        if isinstance(w, DenseWorkload) else "sampled rows / tokens",
              "tolerance": "1e-2 * (|ref| + rms(ref)) against the CPU oracle (2e-2 for the MoE step; quantiser bit-exact)"}
    if line is not None:
        line["parity_check"] = parity

    if default_line and world == 1:
        # ---- the same operands through torch.matmul (cuBLAS) in the same run, and a sustained block of both
        n = args.steps * gps
        c_total, c_unit, _, _ = run.timed(lambda i: w.cublas_step(i), args.warmup * gps, n, clocks=False)
        line["cublas_same_run"] = {"tflops": w.kernel_flops / (c_unit * 1e-3) / 1e12, "ms": c_unit,
                                   "ours_over_cublas": c_unit / unit_ms,
                                   "how": "torch.matmul(A, B^T view, out=C) on the same rotating operand sets, same launch count"}
        n_sus = int(1800.0 / unit_ms) + 1
        s_total, s_unit, s_ck, _ = run.timed(lambda i: w.step(i, dist), 8, n_sus)
        cs_total, cs_unit, cs_ck, _ = run.timed(lambda i: w.cublas_step(i), 8, n_sus)
        line["sustained"] = {"value": w.flops * n_sus / (s_total * 1e-3) / 1e12, "unit": "TFLOP/s", "seconds": s_total * 1e-3,
                             "launches": n_sus, "sm_mhz_median": s_ck["sm_mhz"], "power_w_max": s_ck.get("power_w_max"),
                             "reasons": s_ck["reasons"], "clock_samples": s_ck.get("samples"),
                             "frac_of_measured_sustained_cublas": w.flops * n_sus / (s_total * 1e-3) / 1e12 / peaks["bf16_tflops_sustained"],
                             "cublas_same_run": {"tflops": w.flops * n_sus / (cs_total * 1e-3) / 1e12,
                                                 "sm_mhz_median": cs_ck["sm_mhz"], "power_w_max": cs_ck.get("power_w_max")}}
    del w
    release()

    if default_line:
        moe = moe_block(args, run, nccl=False)
        moe_nccl = moe_block(args, run, nccl=True) if world > 1 else None
        if line is not None:
            line["moe"] = moe
            if moe_nccl is not None:
                line["moe_nccl"] = moe_nccl

    if default_line and world == 1:
        items = []
        for name in EXTRA_WORKLOADS:
            xw = make_workload(name, args, dev, rank, world)
            # about a quarter of a second of launches, timed one by one
            _, est, _, _ = run.timed(lambda i: xw.step(i, dist), 3, 5, clocks=False)
            n = max(20, min(4000, int(250.0 / max(est, 1e-3))))
            total, unit, ck, nl = run.timed(lambda i: xw.step(i, dist), 3, n)
            ok, err = xw.parity_check(dist)
            lib_run = None
            if hasattr(xw, "cublas_step"):
                # the vendor library on the same operands in the same run (context, not a denominator)
                try:
                    _, lib_unit, _, _ = run.timed(lambda i: xw.cublas_step(i), 3, n, clocks=False)
                    lib_run = {"ms": lib_unit, "ours_over_library": lib_unit / unit,
                               "how": "torch._scaled_mm (cuBLASLt, row-wise scales)" if xw.fp8 else "torch.matmul (cuBLAS)"}
                except Exception as exc:      # a torch build without this cuBLASLt path
                    lib_run = {"unavailable": str(exc).splitlines()[0][:200]}
            # the same launches with nothing recorded between them: what a chain of such kernels costs per link (launch
            # gaps included; kernels that start while their predecessor drains get to show it)
            _, b2b, _, _ = run.timed(lambda i: xw.step(i, dist), 3, n, clocks=False, per_call_events=False)
            back_to_back = {"ms": b2b}
            if lib_run is not None and "ms" in lib_run:
                _, lib_b2b, _, _ = run.timed(lambda i: xw.cublas_step(i), 3, n, clocks=False, per_call_events=False)
                back_to_back.update({"library_ms": lib_b2b, "ours_over_library": lib_b2b / b2b})
            flops = xw.kernel_flops if name != "mxfp4_quant" else 0.0
            items.append({"workload": f"{name}: {xw.label}", "value": (flops / (unit * 1e-3) / 1e12) if flops else None,
                          "unit": "TFLOP/s", "kernel_ms": unit, "launches": n, "gpu_launches": nl,
                          "roofline": roofline_of(name, xw, unit, total * 1e-3, peaks, 1), "clocks": ck,
                          "parity_check": {"ok": ok, "max_err": err}, "library_same_run": lib_run,
                          "back_to_back": back_to_back})
            del xw
            release()
        line["workloads"] = items

    if line is not None:
        if not args.no_cpu_baseline and world == 1:
            if args.workload == "moe":
                M, N, K = 2048, MOE["hidden"], 2 * MOE["ffn"]
            else:
                M, N, K = wl["M"], wl["N"], wl["K"]
            tf, rows, dt = cpu_reference_tflops(M, N, K, TORCH_DTYPES.get(wl["dtype"], torch.bfloat16), target_seconds=12.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": f"torch.matmul (fp32 accumulate) of {rows} of {M} rows of A against the "
                                              f"full {K}x{N} B, repeated for {dt:.1f} s in total"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
