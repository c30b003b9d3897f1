"""The MoE step's device-side dispatch plan and the single-GPU form of the peer-memory path, against the torch index
arithmetic that specifies the plan (tritonblas_b200.distributed.plan_peer_dispatch) and the CPU oracle of the step.
The reference has no MoE path: parity unpinned by construction; tolerance 2e-2 * (|ref| + rms) for the chained bf16
GEMMs plus one bf16 ulp of the largest reference value (an intermediate of that size may round the other way), index
outputs exact."""
import ctypes

import pytest
import torch

import tritonblas_b200 as tb
from tritonblas_b200 import _lib
from tritonblas_b200 import distributed as tbd
from oracle import moe_oracle

pytestmark = pytest.mark.gpu


def _zipf_ids(T, E, topk, seed, dtype=torch.int64):
    g = torch.Generator().manual_seed(seed)
    p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.1
    p = (p / p.sum())[torch.randperm(E, generator=g)]
    return torch.multinomial(p.expand(T, E), topk, replacement=False, generator=g).to(dtype)


@pytest.mark.parametrize("world,E,T,topk,dtype", [(1, 64, 16384, 8, torch.int64), (4, 16, 37, 3, torch.int32),
                                                  (8, 64, 2048, 8, torch.int64), (2, 1024, 300, 4, torch.int32),
                                                  (1, 8, 1, 2, torch.int64)])
def test_plan_kernels_match_the_index_arithmetic_specification(world, E, T, topk, dtype):
    """All ranks of an expert-parallel group emulated on one GPU: counts equal a histogram; group offsets equal the
    specification's; every (source rank, expert) segment of every receive buffer is filled exactly once."""
    lib = _lib.lib
    stream = _lib.current_stream_ptr()
    ids = [_zipf_ids(T, E, topk, 100 + r, dtype).cuda() for r in range(world)]
    counts_all = torch.zeros(world, E, dtype=torch.int32, device="cuda")
    for r in range(world):
        counts_all[r].fill_(-7)          # the call clears its output
        _lib.check(lib.tb_moe_count(ctypes.c_void_p(ids[r].data_ptr()), int(dtype == torch.int64), T * topk, E, None,
                                    ctypes.c_void_p(counts_all[r].data_ptr()), stream), "tb_moe_count")
        assert torch.equal(counts_all[r].cpu().long(), torch.bincount(ids[r].flatten().cpu().long(), minlength=E))
    epr = E // world
    cap = int(counts_all.sum())
    landed = [torch.zeros(cap, dtype=torch.int32) for _ in range(world)]
    for r in range(world):
        spec = tbd.plan_peer_dispatch(ids[r].cpu(), counts_all.cpu().long(), r)
        pair_rank = torch.empty(T * topk, dtype=torch.int32, device="cuda")
        pair_row = torch.empty(T * topk, dtype=torch.int64, device="cuda")
        offs = torch.empty(epr + 1, dtype=torch.int32, device="cuda")
        cursor = torch.full((E,), 123, dtype=torch.int32, device="cuda")
        for _ in range(2):               # the cursor is cleared by the call: a second call gives a valid plan again
            _lib.check(lib.tb_moe_plan(ctypes.c_void_p(ids[r].data_ptr()), int(dtype == torch.int64), T * topk, E, None, world, r,
                                       ctypes.c_void_p(counts_all.data_ptr()), ctypes.c_void_p(cursor.data_ptr()), cap,
                                       ctypes.c_void_p(pair_rank.data_ptr()), ctypes.c_void_p(pair_row.data_ptr()),
                                       ctypes.c_void_p(offs.data_ptr()), None, topk, stream), "tb_moe_plan")
        assert offs.cpu().tolist() == spec.group_offsets.tolist()
        assert torch.equal(pair_rank.cpu(), spec.pair_rank)
        # same rows as the specification per expert, in any order
        flat = ids[r].flatten().cpu().long()
        got, want = pair_row.cpu(), spec.pair_row
        for e in torch.unique(flat).tolist():
            sel = flat == e
            assert torch.equal(torch.sort(got[sel]).values, torch.sort(want[sel]).values), (r, e)
        for d, row in zip(pair_rank.cpu().tolist(), got.tolist()):
            landed[d][row] += 1
    for d in range(world):
        used = int(counts_all[:, d * epr:(d + 1) * epr].sum())
        assert bool((landed[d][:used] == 1).all()) and bool((landed[d][used:] == 0).all())


def _experts(E, H, F, seed):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(E, 2 * F, H, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w2 = (torch.randn(E, H, F, generator=g) * 0.05).to(torch.bfloat16).cuda()
    return w1, w2


@pytest.mark.parametrize("gather_rows", [False, True])
@pytest.mark.parametrize("E,H,F,T,topk", [(8, 256, 128, 64, 2), (64, 512, 256, 1000, 8), (16, 1024, 384, 333, 4)])
def test_single_gpu_moe_step_matches_oracle(E, H, F, T, topk, gather_rows):
    w1, w2 = _experts(E, H, F, E + T)
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    ids = _zipf_ids(T, E, topk, 7).cuda()
    wts = torch.rand(T, topk, generator=g).cuda()
    moe = tbd.PeerMemoryMoE(w1, w2, E, capacity=T * topk, gather_rows=gather_rows)
    for _ in range(2):
        out, plan = moe.forward(x, ids, wts)
        toks = list(range(0, T, max(1, T // 48)))
        ref = moe_oracle.moe_ffn_ref(x, ids, wts, lambda e: w1[e], lambda e: w2[e], toks)
        got = out[torch.tensor(toks, device="cuda")].float().cpu()
        rms = ref.pow(2).mean().sqrt().item()
        err = (got - ref).abs()
        assert bool((err <= 2e-2 * ref.abs() + 2e-2 * rms + 2 ** -8 * ref.abs().max()).all()), err.max().item()
    assert int(moe.overflow.item()) == 0 and tb.device_status() == 0
    assert int(plan.group_offsets[-1]) == T * topk


def test_capacity_below_the_routing_drops_rows_without_reaching_past_the_buffers():
    """capacity smaller than the routed rows: the dispatch drops and counts the tail rows, the grouped GEMMs' offsets end
    exactly at the buffer's last row, the combine step skips the dropped pairs, and tokens none of whose pairs were dropped
    still match the oracle."""
    E, H, F, T, topk = 8, 256, 128, 200, 2
    w1, w2 = _experts(E, H, F, 3)
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    ids = _zipf_ids(T, E, topk, 9).cuda()
    wts = torch.rand(T, topk, generator=g).cuda()
    cap = T * topk - 37
    moe = tbd.PeerMemoryMoE(w1, w2, E, capacity=cap)
    out, plan = moe.forward(x, ids, wts)
    torch.cuda.synchronize()
    assert int(moe.overflow.item()) == 37
    assert int(plan.group_offsets[-1]) == cap
    kept = (plan.pair_row.view(T, topk) < cap).all(dim=1).cpu()
    toks = [t for t in range(T) if bool(kept[t])][:40]
    ref = moe_oracle.moe_ffn_ref(x, ids, wts, lambda e: w1[e], lambda e: w2[e], toks)
    got = out[torch.tensor(toks, device="cuda")].float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    assert bool(((got - ref).abs() <= 2e-2 * ref.abs() + 2e-2 * rms + 2 ** -8 * ref.abs().max()).all())
    assert torch.isfinite(out.float()).all() and tb.device_status() == 0


def test_balanced_placement_single_gpu_results_do_not_depend_on_the_layout_order():
    """expert_place permutes where experts live (and the order of this rank's weights); the MoE output is the same
    function of the tokens, so it matches the oracle evaluated with the experts' own weights."""
    E, H, F, T, topk = 16, 256, 128, 300, 4
    w1, w2 = _experts(E, H, F, 21)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).cuda()
    ids = _zipf_ids(T, E, topk, 13).cuda()
    wts = torch.rand(T, topk, generator=g).cuda()
    load = torch.bincount(ids.flatten().cpu(), minlength=E)
    place = tbd.balanced_expert_placement(load, 4)
    assert sorted(place.tolist()) == list(range(E))
    per_rank = torch.zeros(4, dtype=torch.int64).index_add_(0, (place // (E // 4)).long(), load)
    contiguous = load.reshape(4, -1).sum(1)
    assert per_rank.max() <= contiguous.max()
    inv = torch.empty(E, dtype=torch.int64)
    inv[place.long()] = torch.arange(E)
    moe = tbd.PeerMemoryMoE(w1[inv.cuda()].contiguous(), w2[inv.cuda()].contiguous(), E, capacity=T * topk, expert_place=place)
    out, _ = moe.forward(x, ids, wts)
    toks = list(range(0, T, 7))
    ref = moe_oracle.moe_ffn_ref(x, ids, wts, lambda e: w1[e], lambda e: w2[e], toks)
    got = out[torch.tensor(toks, device="cuda")].float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    assert bool(((got - ref).abs() <= 2e-2 * ref.abs() + 2e-2 * rms + 2 ** -8 * ref.abs().max()).all())
