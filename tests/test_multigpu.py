"""Two-rank NCCL run of the column-sharded GEMM (NCCL all-gather and the fused epilogue push) and of the expert-parallel
MoE path. Needs two GPUs: skipped otherwise. Runs as child processes, one per GPU."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["TB_ROOT"])
import tritonblas_b200 as tb
from tritonblas_b200 import distributed as tbd
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
g = torch.Generator().manual_seed(0)
M, N, K = 512, 1024, 768
a = (torch.randn(M, K, generator=g) * 0.1).to(torch.bfloat16).to(dev)
b = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(dev)       # (N, K): K-contiguous
lo, hi = tbd.shard_range(N, world, rank)
layer = tbd.ColumnShardedGemm(b[lo:hi].contiguous())
ref = a.float() @ b.float().T
c = tbd.ColumnShardedGemm.as_matrix(layer.forward(a)).float()
assert torch.allclose(c, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item()), "nccl all-gather path"
layer.enable_fused_gather(M)
for _ in range(2):
    c2 = tbd.ColumnShardedGemm.as_matrix(layer.forward_fused(a)).float()
    assert torch.allclose(c2, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item()), "fused push path"
for frac in (0.4, 1.0):        # the last tiles of the launch cross NVLink from a side stream
    for _ in range(2):
        g3 = layer.forward_fused(a, overlap_tail=frac)
        layer.wait_gathered()
        c4 = tbd.ColumnShardedGemm.as_matrix(g3).float()
        assert torch.allclose(c4, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item()), "fused push with tail copy"
for _ in range(2):             # the whole block by asynchronous peer copies on side streams
    g4 = layer.forward_fused(a, overlap_tail=1.0, tail_by_copy_engine=True)
    layer.wait_gathered()
    c5 = tbd.ColumnShardedGemm.as_matrix(g4).float()
    assert torch.allclose(c5, ref, rtol=1e-2, atol=1e-2 * ref.abs().max().item()), "gathered by peer copies"
# first row groups of tiles from the epilogue, the rows of the last ones by peer copies; a taller product so that the tile
# order has several groups, and the buffers poisoned before every call so that a row nobody sent cannot pass
M2, K2 = 4096, 256
a2 = (torch.randn(M2, K2, generator=g) * 0.1).to(torch.bfloat16).to(dev)
b2 = (torch.randn(N, K2, generator=g) * 0.1).to(torch.bfloat16).to(dev)
layer2 = tbd.ColumnShardedGemm(b2[lo:hi].contiguous())
buf2 = layer2.enable_fused_gather(M2)
layer2._fused_selector.override(group_m=4)
ref2 = a2.float() @ b2.float().T
for frac in (0.3, 0.5, 0.8):
    first_tile, first_row = layer2._tail_split(a2, layer2.b_shard_t, frac)
    assert 0 < first_row < M2 and first_tile > 0, (frac, first_tile, first_row)
    for _ in range(2):
        buf2.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        g5 = layer2.forward_fused(a2, overlap_tail=frac, tail_by_copy_engine=True)
        layer2.wait_gathered()
        c6 = tbd.ColumnShardedGemm.as_matrix(g5).float()
        assert torch.allclose(c6, ref2, rtol=1e-2, atol=1e-2 * ref2.abs().max().item()), ("epilogue pushes + peer copies", frac)
        torch.cuda.synchronize()
        dist.barrier()
# expert-parallel MoE against a single-device evaluation of the same experts
E, H, F, T, topk = 8, 256, 128, 64, 2
w1 = (torch.randn(E, 2 * F, H, generator=g) * 0.1).to(torch.bfloat16).to(dev)
w2 = (torch.randn(E, H, F, generator=g) * 0.1).to(torch.bfloat16).to(dev)
xs = torch.randn(world, T, H, generator=g).to(torch.bfloat16).to(dev)
ids = torch.stack([torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]) for _ in range(world)]).to(dev)
wts = torch.rand(world, T, topk, generator=g).to(dev)
epr = E // world
moe = tbd.ExpertParallelMoE(w1[rank * epr:(rank + 1) * epr].contiguous(), w2[rank * epr:(rank + 1) * epr].contiguous(), E)
out, _ = moe.forward(xs[rank], ids[rank], wts[rank])
ref = torch.zeros(T, H, device=dev)
for t in range(T):
    for j in range(topk):
        e = int(ids[rank, t, j])
        h = xs[rank, t].float() @ w1[e].float().T
        act = (torch.nn.functional.silu(h[:F]) * h[F:]).to(torch.bfloat16).float()
        ref[t] += wts[rank, t, j] * (act @ w2[e].float().T).to(torch.bfloat16).float()
assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item()), "expert-parallel MoE"
peer = tbd.PeerMemoryMoE(w1[rank * epr:(rank + 1) * epr].contiguous(), w2[rank * epr:(rank + 1) * epr].contiguous(), E,
                         capacity=world * T * topk)
for _ in range(2):
    out2, _ = peer.forward(xs[rank], ids[rank], wts[rank])
    assert torch.allclose(out2.float(), ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item()), "peer-memory MoE"
assert int(peer.overflow.item()) == 0
# unaligned shard (K not a multiple of 8): the CUDA-core kernel must fan the tiles out to the peers as well
K2 = 100
a2 = (torch.randn(64, K2, generator=g) * 0.1).to(torch.bfloat16).to(dev)
b2 = (torch.randn(256, K2, generator=g) * 0.1).to(torch.bfloat16).to(dev)
lo2, hi2 = tbd.shard_range(256, world, rank)
layer2 = tbd.ColumnShardedGemm(b2[lo2:hi2].contiguous())
layer2.enable_fused_gather(64)
c3 = tbd.ColumnShardedGemm.as_matrix(layer2.forward_fused(a2)).float()
ref3 = a2.float() @ b2.float().T
assert torch.allclose(c3, ref3, rtol=1e-2, atol=1e-2 * ref3.abs().max().item()), "fused push from the CUDA-core kernel"
assert tb.device_status(rank) == 0
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
"""


def test_two_rank_sharded_gemm_fused_push_and_moe():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TB_ROOT=ROOT, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<timed out>"
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n----\n".join(o[-3000:] for o in outs)
