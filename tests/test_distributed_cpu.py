"""Host-side logic of the two multi-GPU paths on CPU: world_size-2 gloo ranks, with torch.matmul standing in for the
CUDA GEMM entry points (only the partitioning, routing and collective plumbing is under test here)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tritonblas_b200 import distributed as tbd


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _grouped_cpu(x, w, offs, out=None):
    y = torch.zeros(x.shape[0], w.shape[1], dtype=x.dtype)
    for e in range(w.shape[0]):
        lo, hi = int(offs[e]), int(offs[e + 1])
        y[lo:hi] = (x[lo:hi].float() @ w[e].float().T).to(x.dtype)
    return y


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        # ---- column-sharded GEMM + all-gather
        M, N, K = 24, 32, 40
        a = torch.randn(M, K, generator=g)
        b = torch.randn(K, N, generator=g)
        lo, hi = tbd.shard_range(N, world, rank)
        layer = tbd.ColumnShardedGemm(b[:, lo:hi].T.contiguous(), matmul_fn=lambda x, y, out=None: torch.matmul(x, y))
        c = tbd.ColumnShardedGemm.as_matrix(layer.forward(a))
        assert torch.allclose(c, a @ b, atol=1e-4), "sharded GEMM"
        # ---- expert-parallel MoE
        E, H, F, T, topk = 8, 16, 12, 10, 3
        w1 = torch.randn(E, 2 * F, H, generator=g) * 0.2
        w2 = torch.randn(E, H, F, generator=g) * 0.2
        xs = torch.randn(world, T, H, generator=g)
        ids = torch.stack([torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]) for _ in range(world)])
        wts = torch.rand(world, T, topk, generator=g)
        epr = E // world
        moe = tbd.ExpertParallelMoE(w1[rank * epr:(rank + 1) * epr], w2[rank * epr:(rank + 1) * epr], E, grouped_fn=_grouped_cpu)
        out, plan = moe.forward(xs[rank], ids[rank], wts[rank])
        ref = torch.zeros(T, H)
        for t in range(T):
            for j in range(topk):
                e = int(ids[rank, t, j])
                h = xs[rank, t] @ w1[e].T
                ref[t] += wts[rank, t, j] * ((torch.nn.functional.silu(h[:F]) * h[F:]) @ w2[e].T)
        assert torch.allclose(out, ref, atol=1e-4), "expert-parallel MoE"
        assert int(plan.group_offsets[-1]) == int(sum(plan.recv_splits))
        results[rank] = "ok"
    except Exception as exc:  # surfaced by the parent
        results[rank] = repr(exc)
    finally:
        dist.destroy_process_group()


def test_sharded_gemm_and_expert_parallel_moe_two_ranks():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}, dict(results)


def test_shard_range_covers_axis():
    for n, world in ((8192, 8), (10, 4), (7, 2), (3, 4)):
        spans = [tbd.shard_range(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))


def test_single_rank_plan_is_identity_routing():
    ids = torch.tensor([[1, 0], [0, 2], [2, 1]])
    plan = tbd.plan_dispatch(ids, 4)
    assert plan.regroup_idx is None and plan.group_offsets.tolist() == [0, 2, 4, 6, 6]
    x = torch.arange(6.0).reshape(3, 2)
    rows = tbd.dispatch(x, 2, plan)
    assert rows.shape == (6, 2)
    back = tbd.combine(rows, torch.ones(3, 2), plan)
    assert torch.allclose(back, 2 * x)


def test_peer_dispatch_plan_places_every_row_once_and_expert_major():
    """The index arithmetic of the peer-memory MoE path, emulated for 4 ranks in one process: after every rank has
    "written" its rows, each rank's receive buffer holds its experts back to back, each expert's rows complete, and the
    combine indices point back at the row that carries the pair's token."""
    world, E, T, topk = 4, 16, 37, 3
    g = torch.Generator().manual_seed(5)
    ids = [torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]) for _ in range(world)]
    counts_all = torch.stack([torch.bincount(i.flatten(), minlength=E) for i in ids])
    plans = [tbd.plan_peer_dispatch(ids[r], counts_all, r) for r in range(world)]
    epr = E // world
    cap = int(counts_all.sum())
    token_tag = [torch.full((cap,), -1, dtype=torch.int64) for _ in range(world)]     # what landed where: (src, token)
    expert_tag = [torch.full((cap,), -1, dtype=torch.int64) for _ in range(world)]
    for r, p in enumerate(plans):
        flat = ids[r].flatten()
        sort_idx = torch.argsort(flat, stable=True)
        for i in range(p.src_token.numel()):
            d, row = int(p.dest_rank[i]), int(p.dest_row[i])
            assert token_tag[d][row] == -1, "two rows written to the same place"
            token_tag[d][row] = r * 1000 + int(p.src_token[i])
            expert_tag[d][row] = int(flat[sort_idx[i]])
    for d in range(world):
        offs = plans[d].group_offsets.tolist()
        assert offs[-1] == int(counts_all[:, d * epr:(d + 1) * epr].sum())
        for e in range(epr):
            seg = expert_tag[d][offs[e]:offs[e + 1]]
            assert (seg == d * epr + e).all()
        assert (token_tag[d][offs[-1]:] == -1).all()
    for r, p in enumerate(plans):
        for f in range(T * topk):
            d, row = int(p.pair_rank[f]), int(p.pair_row[f])
            assert token_tag[d][row] == r * 1000 + f // topk
            assert expert_tag[d][row] == int(ids[r].flatten()[f])


def test_peer_dispatch_plan_clamps_group_offsets_to_capacity():
    """A receive buffer smaller than the routing needs: the dispatch kernel drops rows at or beyond `capacity`; the group
    offsets handed to the grouped GEMM are clamped to it (never past the buffer, still ascending), and the pairs whose row
    was dropped are exactly those the combine kernel skips (row >= capacity)."""
    world, E, T, topk = 2, 8, 50, 2
    g = torch.Generator().manual_seed(6)
    ids = [torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)]) for _ in range(world)]
    counts_all = torch.stack([torch.bincount(i.flatten(), minlength=E) for i in ids])
    epr = E // world
    for r in range(world):
        need = int(counts_all[:, r * epr:(r + 1) * epr].sum())
        cap = need - 17
        full = tbd.plan_peer_dispatch(ids[r], counts_all, r)
        clamped = tbd.plan_peer_dispatch(ids[r], counts_all, r, capacity=cap)
        offs = clamped.group_offsets.tolist()
        assert offs[0] == 0 and offs[-1] == cap and all(a <= b for a, b in zip(offs, offs[1:]))
        assert offs == [min(o, cap) for o in full.group_offsets.tolist()]
        assert torch.equal(clamped.dest_row, full.dest_row)           # rows keep their places; the kernels drop the tail
    dropped = sum(int(((tbd.plan_peer_dispatch(ids[r], counts_all, r).dest_row >= int(counts_all[:, d * epr:(d + 1) * epr].sum()) - 17)
                       & (tbd.plan_peer_dispatch(ids[r], counts_all, r).dest_rank == d)).sum())
                  for r in range(world) for d in range(world))
    assert dropped == 17 * world


def test_balanced_expert_placement_evens_out_the_rows_per_rank():
    E, topk, T = 64, 8, 4096
    g = torch.Generator().manual_seed(77)
    p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.1
    p = (p / p.sum())[torch.randperm(E, generator=g)]
    ids = torch.multinomial(p.expand(T, E), topk, replacement=False, generator=g)
    load = torch.bincount(ids.flatten(), minlength=E)
    for world in (2, 4, 8):
        place = tbd.balanced_expert_placement(load, world)
        epr = E // world
        assert sorted(place.tolist()) == list(range(E))
        per_rank = torch.zeros(world, dtype=torch.int64).index_add_(0, (place // epr).long(), load)
        contiguous = load.reshape(world, epr).sum(1)
        mean = load.sum().item() / world
        assert per_rank.max().item() <= contiguous.max().item()
        assert per_rank.max().item() / mean < 1.25
    # the single-rank plan honours a placement: experts appear in layout order
    place = tbd.balanced_expert_placement(load, 8)
    plan = tbd.plan_dispatch(ids[:50], E, expert_place=place)
    placed = place.long()[ids[:50].flatten()]
    assert plan.group_offsets.tolist() == [0] + torch.bincount(placed, minlength=E).cumsum(0).tolist()


def test_bench_matmul_csv_schema(tmp_path):
    """The YAML/CSV benchmark tool writes the reference's column set (benchmarks/tritonblas_matmul.py:278-291)."""
    from tritonblas_b200 import bench_matmul as bm
    row = {name: 0 for name in bm.CSV_FIELDS}
    row["active_cus"] = 148
    out = tmp_path / "r.csv"
    bm.write_csv(str(out), [row])
    header = out.read_text().splitlines()[0].split(",")
    assert header == ["active_cus", "m", "n", "k", "mnk", "macro_tile", "bytes", "flops", "tritonblas_gflops", "a_type",
                      "b_type", "c_type", "d_type", "compute_type", "in_dtype", "out_dtype", "init_type", "transA",
                      "transB", "us", "alpha", "beta", "mode"]
    import yaml
    cases = yaml.safe_load(open(bm.__file__.replace("bench_matmul.py", "shapes/baseline.yaml")))
    assert all({"m", "n", "k", "in_dtype", "out_dtype", "transA", "transB"} <= set(c) for c in cases)
    assert all(bm.str_to_dtype(c["in_dtype"]) is not None for c in cases)


def _tile_rows(tile, tiles_m, tiles_n, group_m, block_m):
    """First row of a tile in the kernel's launch order (groups of group_m tile rows, each swept column by column:
    the reference's GROUP_SIZE_M order, kernels/stages/schedule.py:124-145)."""
    width = group_m * tiles_n
    group = tile // width
    first_m = group * group_m
    gsz = min(tiles_m - first_m, group_m)
    return (first_m + (tile - group * width) % gsz) * block_m


def test_tail_split_of_the_gathered_product_follows_the_tile_order():
    """Splitting a product between epilogue pushes (tiles below `first_tile`) and row copies (rows from `first_row` on):
    every tile below the limit lies wholly above the first copied row and every other tile wholly below it."""
    import tritonblas_b200 as tb
    for (m, n, k, group_m, frac) in [(8192, 2048, 8192, 0, 0.5), (8192, 1024, 8192, 0, 0.3), (4096, 512, 256, 4, 0.8),
                                     (4096, 512, 256, 4, 0.3), (2304, 768, 512, 2, 0.5), (512, 512, 256, 0, 0.5)]:
        layer = tbd.ColumnShardedGemm(torch.zeros(n, k, dtype=torch.bfloat16), matmul_fn=lambda *a: None)
        sel = tb.OrigamiMatmulSelector(m, n, k, torch.bfloat16, torch.bfloat16, torch.bfloat16, torch.device("cpu"), max_halves=1)
        if group_m:
            sel.override(group_m=group_m)
        layer._fused_selector = sel
        a = torch.zeros(m, k, dtype=torch.bfloat16)
        first_tile, first_row = layer._tail_split(a, layer.b_shard_t, frac)
        cfg = sel.config_for(False, False)
        tiles_m, tiles_n = -(-m // cfg.block_m), -(-n // (cfg.block_n * max(cfg.n_halves, 1)))
        gm = cfg.group_m if cfg.group_m > 0 else 8
        total = tiles_m * tiles_n
        assert 0 < first_tile <= total and 0 < first_row <= m
        for t in range(total):
            r0 = _tile_rows(t, tiles_m, tiles_n, gm, cfg.block_m)
            if t < first_tile:
                assert r0 + cfg.block_m <= first_row or first_row == m, (m, n, t, r0, first_row)
            else:
                assert r0 >= first_row, (m, n, t, r0, first_row)
        if -(-tiles_m // gm) >= 2:
            assert first_tile < total and first_row < m        # something is left for the copies
