"""Egress bandwidth of SM-issued stores into a peer GPU's memory, by contiguous run length: the rate that bounds the fused
GEMM + all-gather (every tile of C is stored to P - 1 peers) and the MoE dispatch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m tritonblas_b200.peer_bandwidth

Every rank stores into its right-hand neighbour's symmetric-memory buffer at the same time (both directions of every link
are busy, as in an all-gather); rank 0 prints GB/s per run length for the peer buffer and for its own memory, and, with
more than two ranks, the aggregate rate when every rank stores into ALL its peers at once (one launch per peer, each on
its own stream), which is what an all-gather by stores does. Rows are 16 KB apart, the pitch of a row of C with N = 8192
bf16 columns. Ordinary stores only (no TMA, no multicast).
"""
import ctypes
import os

os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

import torch
import torch.distributed as dist


def measure(run_lengths=(128, 256, 512, 2048, 16384), grids=((148, 128), (148, 512)), buffer_mb=256, pitch=16384):
    import torch.distributed._symmetric_memory as symm_mem
    from tritonblas_b200 import _lib
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    nbytes = buffer_mb << 20
    buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
    handle = symm_mem.rendezvous(buf, group=dist.group.WORLD)
    targets = (("peer", int(handle.buffer_ptrs[(rank + 1) % world])), ("local", int(handle.buffer_ptrs[rank])))
    stream = _lib.current_stream_ptr(dev)
    results = []
    for name, ptr in targets:
        for run in run_lengths:
            for blocks, threads in grids:
                rows = min((128 << 20) // run, nbytes // pitch)
                passes = max(1, (64 << 20) // (rows * run))
                total = rows * run * passes

                def launch():
                    _lib.check(_lib.lib.tb_peer_store_probe(ctypes.c_void_p(ptr), pitch, run, rows, blocks, threads, passes, stream),
                               "tb_peer_store_probe")
                for _ in range(2):
                    launch()
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(8):
                    launch()
                e1.record()
                torch.cuda.synchronize()
                results.append((name, run, blocks, threads, total / (e0.elapsed_time(e1) / 8) / 1e6))
                dist.barrier()
    if world > 2:
        # every peer at once: one launch per peer on its own stream; aggregate egress of this rank
        peers = [int(handle.buffer_ptrs[r]) for r in range(world) if r != rank]
        streams = [torch.cuda.Stream(dev) for _ in peers]
        for run in run_lengths:
            rows = min((128 << 20) // run, nbytes // pitch)
            passes = max(1, (64 << 20) // (rows * run))
            total = rows * run * passes * len(peers)

            def launch_all():
                for ptr, st in zip(peers, streams):
                    _lib.check(_lib.lib.tb_peer_store_probe(ctypes.c_void_p(ptr), pitch, run, rows, 148, 256, passes,
                                                            ctypes.c_void_p(st.cuda_stream)), "tb_peer_store_probe")
            for _ in range(2):
                launch_all()
            torch.cuda.synchronize()
            dist.barrier()
            main = torch.cuda.current_stream()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for st in streams:
                st.wait_stream(main)
            for _ in range(4):
                launch_all()
            for st in streams:
                main.wait_stream(st)
            e1.record()
            torch.cuda.synchronize()
            results.append((f"all {len(peers)} peers", run, 148, 256, total / (e0.elapsed_time(e1) / 4) / 1e6))
            dist.barrier()
    return results


def main():
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    results = measure()
    if rank == 0:
        for name, run, blocks, threads, gbs in results:
            print(f"{name:11s} run {run:6d} B  grid {blocks:4d} x {threads:3d} : {gbs:8.1f} GB/s")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
