"""Rate at which the SMs pull a K-major matrix out of HBM with the GEMM's own operand-loader pattern (TMA boxes of
box_rows rows x 128 bytes, rows one pitch apart, K walked in 128-byte steps, one CTA per SM) and nothing else going on:
the ceiling of the streaming phase of the decode-shaped GEMMs (few rows of activations against a wide weight matrix).

    python -m tritonblas_b200.hbm_stream [--rows 86016] [--k 8192]

Prints one line per (ring depth, box rows) with GB/s from CUDA events (best of 5 launches); the matrix defaults to three
times the 28672 x 8192 bf16 decode weight (1.4 GB, eleven times the L2).
"""
import argparse
import ctypes
import json

import torch


def measure(rows=86016, k=8192, programs=None, configs=((4, 128), (6, 128), (8, 128), (10, 128), (12, 128), (4, 256), (6, 256),
                                                          (16, 64), (24, 64))):
    from tritonblas_b200 import _lib, device_status
    dev = torch.device("cuda", torch.cuda.current_device())
    programs = programs or torch.cuda.get_device_properties(dev).multi_processor_count
    w = torch.ones(rows, k, dtype=torch.bfloat16, device=dev)
    stream = _lib.current_stream_ptr(dev)
    out = []
    for stages, box_rows in configs:
        streamed_rows = rows // box_rows * box_rows

        def launch():
            _lib.check(_lib.lib.tb_tma_stream_probe(ctypes.c_void_p(w.data_ptr()), rows, k * 2, k * 2, stages, box_rows,
                                                    programs, stream), "tb_tma_stream_probe")
        launch()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            launch()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        out.append({"stages": stages, "box_rows": box_rows, "in_flight_kb_per_sm": stages * box_rows * 128 // 1024,
                    "ms": round(best, 4), "gb_s": round(streamed_rows * k * 2 / best / 1e6, 1), "programs": programs,
                    "status": device_status()})
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=86016)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--programs", type=int, default=0)
    a = ap.parse_args()
    for line in measure(a.rows, a.k, a.programs or None):
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
