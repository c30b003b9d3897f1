"""The two multi-GPU paths of the GEMM family, one process per GPU over torch.distributed (NCCL on GPUs):

  * column-sharded weight GEMM: every rank holds A and a contiguous block of B's columns, computes its block of C and the
    ranks all-gather C (tensor-parallel column split);
  * expert-parallel MoE projections: tokens start data-parallel, an all-to-all sends every (token, expert) row to the
    rank that owns the expert, grouped GEMMs run locally, a second all-to-all returns the rows.

The reference is a single-GPU library (its only collectives are background traffic in benchmarks/overlap.py:221-253), so
the semantics here are those of the dense / grouped contracts applied per shard. `matmul_fn` / `grouped_fn` default to
this package's CUDA kernels; the CPU tests of the partition and routing logic pass stand-ins for them.
"""
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def shard_range(n: int, world: int, rank: int):
    """Contiguous [start, stop) of an axis of length n owned by `rank`; earlier ranks take the remainder."""
    base, rem = divmod(n, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


class ColumnShardedGemm:
    """C = A @ B with B split by columns over the ranks of `group`.

    `b_shard_t` is this rank's block of B stored (n_local, K), K-contiguous. forward(a) returns C as a
    (world, M, n_local) tensor (rank r's columns in slice r) when all shards have equal width, which is the gathered
    layout NCCL produces without any extra copy; `as_matrix` materialises the (M, N) matrix when a caller needs it.
    """

    def __init__(self, b_shard_t: torch.Tensor, group=None, matmul_fn: Optional[Callable] = None):
        self.b_shard_t = b_shard_t
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if matmul_fn is None:
            from .matmul import matmul as matmul_fn
        self.matmul_fn = matmul_fn
        self.tail_stream = None          # side stream of forward_fused(overlap_tail > 0)
        self._tail_done = None
        self._peer_views = None          # this rank's block inside every peer's gathered buffer, as tensors
        self._copy_streams = None

    def forward(self, a: torch.Tensor, out_local: Optional[torch.Tensor] = None, gathered: Optional[torch.Tensor] = None):
        c_local = self.matmul_fn(a, self.b_shard_t.T) if out_local is None else (self.matmul_fn(a, self.b_shard_t.T, out_local) or out_local)
        if self.world == 1:
            return c_local.unsqueeze(0)
        if gathered is None:
            gathered = c_local.new_empty(self.world, *c_local.shape)
        # the collective sees the ranks' blocks concatenated along the first axis
        dist.all_gather_into_tensor(gathered.view(self.world * c_local.shape[0], c_local.shape[1]), c_local.contiguous(),
                                    group=self.group)
        return gathered

    def enable_fused_gather(self, m: int, dtype=None, block_n: Optional[int] = None):
        """Allocate the gathered C (world, M, n_local) in symmetric memory and map every peer's copy, so that
        forward_fused() can let the GEMM epilogue write each tile straight into all ranks' buffers over NVLink
        (ordinary stores to peer-mapped memory; no TMA or multicast access to peer memory is involved)."""
        import torch.distributed._symmetric_memory as symm_mem
        dtype = dtype or self.b_shard_t.dtype
        n_local = self.b_shard_t.shape[0]
        group = self.group if self.group is not None else dist.group.WORLD
        self._gathered = symm_mem.empty(self.world, m, n_local, dtype=dtype, device=self.b_shard_t.device)
        self._handle = symm_mem.rendezvous(self._gathered, group=group)
        slot_bytes = m * n_local * self._gathered.element_size()
        # address of MY slot inside every rank's buffer
        self._peer_slots = [int(ptr) + self.rank * slot_bytes for r, ptr in enumerate(self._handle.buffer_ptrs) if r != self.rank]
        from .origami import OrigamiMatmulSelector
        # narrow tiles: their drains, which here also carry the pushes to every peer over NVLink, hide behind the next
        # tile's main loop; a wide tile's drains are exposed (8 GPUs: 3.88 PFLOP/s wide against 4.11 narrow)
        self._fused_selector = OrigamiMatmulSelector(m, n_local, self.b_shard_t.shape[1], self.b_shard_t.dtype,
                                                     self.b_shard_t.dtype, dtype, self.b_shard_t.device, max_halves=1)
        if block_n:
            self._fused_selector.override(block_n=int(block_n))     # tile width of the fused launch (tuning)
        return self._gathered

    def forward_fused(self, a: torch.Tensor, pre_barrier: bool = True, b_shard_t: Optional[torch.Tensor] = None,
                      overlap_tail: float = 0.0, tail_by_copy_engine: bool = False,
                      barrier_on_side_stream: bool = False) -> torch.Tensor:
        """One kernel computes this rank's block of C and pushes it into every rank's gathered buffer; a symmetric-memory
        barrier then orders the ranks. Returns this rank's (world, M, n_local) buffer.

        ``pre_barrier`` makes every rank wait until all ranks have finished reading the previous contents before anyone
        overwrites them. It can be dropped (one barrier less per call) when calls alternate between two or more
        gathered buffers and each buffer is read on this stream before the next call is enqueued: a rank can then only
        start overwriting a buffer after every rank has passed the closing barrier of the call in between, which on each
        rank's stream comes after its reads. ``b_shard_t`` replaces this rank's block of B for one call (same shape).

        ``barrier_on_side_stream``: the launch is as above but the closing barrier runs on ``self.tail_stream``.

        ``overlap_tail`` in (0, 1]: the epilogue pushes only the first tiles; the last ``overlap_tail`` of the tiles are
        copied to the peers, and the closing barrier runs, on a side stream (``self.tail_stream``). The call returns with
        the GEMM enqueued on the current stream: a product enqueued next (one that does not read this gathered buffer)
        starts while this one's last tiles are still crossing NVLink, at the time its own first tiles have nothing to
        send. ``wait_gathered()`` makes the current stream wait until this rank's buffer is complete. The launching stream
        never waits for a barrier in this mode, so a caller that READS the gathered buffers must keep ``pre_barrier=True``
        (every rank arrives there only after its reads of the previous contents are enqueued); products nobody reads in
        between (a throughput run) can drop it when two buffers alternate."""
        from .matmul import persistent_matmul_lt
        if pre_barrier:
            self._handle.barrier(channel=0)      # nobody is still reading the previous contents
        b_t = self.b_shard_t if b_shard_t is None else b_shard_t
        if overlap_tail <= 0.0 and not barrier_on_side_stream:
            persistent_matmul_lt(a, b_t.T, self._gathered[self.rank], self._fused_selector, None, c_copies=self._peer_slots)
            self._handle.barrier(channel=1)      # every rank's pushes have landed
            return self._gathered
        if self.tail_stream is None:
            self.tail_stream = torch.cuda.Stream(a.device)
        main = torch.cuda.current_stream(a.device)
        if self._tail_done is not None:
            main.wait_event(self._tail_done)     # the previous tail copy has read its tiles
        if tail_by_copy_engine and 0.0 < overlap_tail < 1.0:
            # The first row groups of tiles leave from the epilogue, while the product computes; the rows of the last ones
            # (the kernel walks the tiles in groups of group_m tile rows, so a whole number of groups is a contiguous row
            # range of C) by the copy engines, beside the next product.
            first_tile, first_row = self._tail_split(a, b_t, overlap_tail)
            persistent_matmul_lt(a, b_t.T, self._gathered[self.rank], self._fused_selector, None, c_copies=self._peer_slots,
                                 c_copies_tile_limit=first_tile)
            self._copy_rows_to_peers(a.device, main, first_row)
        elif tail_by_copy_engine:
            # The whole block travels by the GPU's copy engines (one asynchronous copy per peer, each on its own stream):
            # no SM is shared with the products that follow on the launching stream. Measured on 4 GPUs: an SM copy
            # kernel beside a GEMM runs at half its stand-alone rate (0.31 against 0.17 ms per block) and slows the GEMM
            # by a fifth (0.235 against 0.19 ms).
            persistent_matmul_lt(a, b_t.T, self._gathered[self.rank], self._fused_selector, None)
            self._copy_rows_to_peers(a.device, main, 0)
        elif overlap_tail > 0.0:
            persistent_matmul_lt(a, b_t.T, self._gathered[self.rank], self._fused_selector, None, c_copies=self._peer_slots,
                                 c_copies_tail_stream=self.tail_stream, c_copies_tail_fraction=overlap_tail)
        else:
            # every tile leaves from the epilogue; only the closing barrier moves to the side stream, so the next product
            # (one that does not read this result) starts without waiting for the other ranks
            persistent_matmul_lt(a, b_t.T, self._gathered[self.rank], self._fused_selector, None, c_copies=self._peer_slots)
            self.tail_stream.wait_stream(main)
        with torch.cuda.stream(self.tail_stream):
            self._handle.barrier(channel=1)      # every rank's pushes, epilogue and tail copy, have landed
            self._tail_done = self.tail_stream.record_event()
        return self._gathered

    def _copy_rows_to_peers(self, device, main, first_row: int):
        """Rows [first_row, M) of this rank's block to every peer's gathered buffer: one asynchronous copy per peer, each
        on a stream of its own, after everything enqueued on ``main`` so far; ``self.tail_stream`` waits for all of them."""
        if self._peer_views is None:
            shape = tuple(self._gathered.shape)
            self._peer_views = [self._handle.get_buffer(r, shape, self._gathered.dtype)[self.rank]
                                for r in range(self.world) if r != self.rank]
            self._copy_streams = [torch.cuda.Stream(device) for _ in self._peer_views]
        ready = main.record_event()
        mine = self._gathered[self.rank]
        for view, st in zip(self._peer_views, self._copy_streams):
            st.wait_event(ready)
            with torch.cuda.stream(st):
                view[first_row:].copy_(mine[first_row:], non_blocking=True)
            self.tail_stream.wait_stream(st)

    def _tail_split(self, a, b_t, fraction: float):
        """(first tile, first row) of the last row groups of tiles, about ``fraction`` of all of them: tiles below the
        first go from the epilogue, rows from the second on by copies. Follows the kernel's tile order (tile index ->
        group of group_m tile rows, swept column by column)."""
        from .matmul import _is_mn_major, _unit_stride_2d
        m, n = a.shape[0], b_t.shape[0]
        cfg = self._fused_selector.config_for(_is_mn_major(_unit_stride_2d(a), 1), _is_mn_major(_unit_stride_2d(b_t.T), 0))
        tile_n = cfg.block_n * max(cfg.n_halves, 1)
        tiles_m, tiles_n = -(-m // cfg.block_m), -(-n // tile_n)
        group_m = cfg.group_m if cfg.group_m > 0 else 8
        groups = -(-tiles_m // group_m)
        if cfg.swap_ab or groups < 2:
            return tiles_m * tiles_n, m             # a single group (or a transposed launch): everything from the epilogue
        tail_groups = min(groups - 1, max(1, round(fraction * groups)))
        head = groups - tail_groups
        return head * group_m * tiles_n, min(head * group_m * cfg.block_m, m)

    def wait_gathered(self):
        """Make the current stream wait for the side stream's tail copy and closing barrier of the last
        ``forward_fused(..., overlap_tail > 0)`` call."""
        if self._tail_done is not None:
            torch.cuda.current_stream().wait_event(self._tail_done)

    @staticmethod
    def as_matrix(gathered: torch.Tensor) -> torch.Tensor:
        world, m, n_local = gathered.shape
        return gathered.permute(1, 0, 2).reshape(m, world * n_local)


@dataclass
class DispatchPlan:
    """Everything the combine step needs to undo a dispatch."""
    sort_idx: torch.Tensor          # (T*topk,) positions of the flattened (token, k) pairs in expert order
    send_counts: torch.Tensor       # (world, experts_per_rank) rows this rank sends, per destination expert
    recv_counts: torch.Tensor       # (world, experts_per_rank) rows this rank receives, per source rank and local expert
    send_splits: List[int]
    recv_splits: List[int]
    regroup_idx: Optional[torch.Tensor]   # received rows (source-major) -> expert-major order
    group_offsets: torch.Tensor     # int32 (experts_per_rank + 1,) row offsets of the expert-major buffer
    regroup_inv: Optional[torch.Tensor] = None   # expert-major -> source-major (inverse of regroup_idx)
    pos: Optional[torch.Tensor] = None           # position of every (token, k) pair in expert order (inverse of sort_idx)


def balanced_expert_placement(expert_load, world: int) -> torch.Tensor:
    """Placement of the experts over ``world`` ranks that evens out the rows per rank: ``place[e]`` is expert e's position
    in the layout order (position q lives on rank q // experts_per_rank as local expert q % experts_per_rank).

    ``expert_load``: rows per expert observed on a calibration batch (any non-negative weights). Greedy longest-processing-
    time assignment with equal cardinality: experts in descending load order each go to the least loaded rank that still
    has a free slot. With a skewed (Zipf) routing distribution the contiguous layout can put several popular experts on one
    rank, whose grouped GEMMs then take a multiple of the mean time; every rank waits for it."""
    load = torch.as_tensor(expert_load).detach().cpu().to(torch.float64).reshape(-1)
    E = load.numel()
    assert E % world == 0, "experts must divide evenly over the ranks"
    epr = E // world
    rank_load, rank_fill = [0.0] * world, [0] * world
    place = torch.empty(E, dtype=torch.int32)
    for e in torch.argsort(load, descending=True, stable=True).tolist():
        r = min((r for r in range(world) if rank_fill[r] < epr), key=lambda q: (rank_load[q], q))
        place[e] = r * epr + rank_fill[r]
        rank_fill[r] += 1
        rank_load[r] += float(load[e])
    return place


def plan_dispatch(topk_ids: torch.Tensor, num_experts: int, group=None, expert_place: Optional[torch.Tensor] = None) -> DispatchPlan:
    """Sort the (token, k) pairs of this rank by expert and exchange per-expert row counts with the other ranks.
    ``expert_place`` maps expert ids to their position in the layout order (see balanced_expert_placement)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    epr = num_experts // world
    flat = topk_ids.reshape(-1).to(torch.int64)
    if expert_place is not None:
        flat = expert_place.to(flat.device).to(torch.int64)[flat]
    sort_idx = torch.argsort(flat, stable=True)
    send_counts = torch.bincount(flat, minlength=num_experts).reshape(world, epr)
    if world > 1:
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
    else:
        recv_counts = send_counts.clone()
    send_splits = send_counts.sum(1).tolist()
    recv_splits = recv_counts.sum(1).tolist()
    # received rows arrive source-major, each source's rows expert-sorted; regroup them expert-major
    per_expert = recv_counts.sum(0)
    group_offsets = torch.zeros(epr + 1, dtype=torch.int32, device=topk_ids.device)
    group_offsets[1:] = per_expert.cumsum(0).to(torch.int32)
    regroup_idx = regroup_inv = None
    pos = torch.empty_like(sort_idx)
    pos[sort_idx] = torch.arange(sort_idx.numel(), device=sort_idx.device)
    if world > 1:
        total = int(sum(recv_splits))
        seg_start_src = (recv_counts.reshape(-1).cumsum(0) - recv_counts.reshape(-1)).reshape(world, epr)   # source-major
        counts_em = recv_counts.T.contiguous()                                                           # (epr, world)
        seg_start_dst = (counts_em.reshape(-1).cumsum(0) - counts_em.reshape(-1)).reshape(epr, world)     # expert-major
        seg_len = counts_em.reshape(-1)
        seg_src = seg_start_src.T.contiguous().reshape(-1)
        seg_id = torch.repeat_interleave(torch.arange(seg_len.numel(), device=seg_len.device), seg_len, output_size=total)
        within = torch.arange(total, device=seg_len.device) - seg_start_dst.reshape(-1)[seg_id]
        regroup_idx = seg_src[seg_id] + within
        regroup_inv = torch.empty_like(regroup_idx)
        regroup_inv[regroup_idx] = torch.arange(total, device=regroup_idx.device)
    return DispatchPlan(sort_idx, send_counts, recv_counts, send_splits, recv_splits, regroup_idx, group_offsets,
                        regroup_inv, pos)


def _gather_rows(x: torch.Tensor, index: torch.Tensor) -> torch.Tensor:
    """x[index] for 2-D x: this library's row-gather kernel for 16-bit CUDA rows of 16-byte multiples, torch otherwise."""
    if not (x.is_cuda and x.element_size() == 2 and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        return x.index_select(0, index)
    import ctypes
    from . import _lib
    index = index.to(torch.int64).contiguous()
    out = x.new_empty(index.numel(), x.shape[1])
    with torch.cuda.device(x.device):
        rc = _lib.lib.tb_moe_gather_rows(ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(index.data_ptr()),
                                         ctypes.c_void_p(out.data_ptr()), out.stride(0), index.numel(), x.shape[1],
                                         _lib.current_stream_ptr(x.device))
    _lib.check(rc, "tb_moe_gather_rows")
    return out


def dispatch(x: torch.Tensor, topk: int, plan: DispatchPlan, group=None) -> torch.Tensor:
    """Rows of x (T, H), replicated topk times and ordered by expert, sent to the experts' owners. Returns the rows this
    rank's experts must process, expert-major (aligned with plan.group_offsets)."""
    rows = _gather_rows(x, plan.sort_idx // topk)
    if plan.regroup_idx is None:
        return rows
    recv = rows.new_empty(int(sum(plan.recv_splits)), x.shape[1])
    dist.all_to_all_single(recv, rows, plan.recv_splits, plan.send_splits, group=group)
    return _gather_rows(recv, plan.regroup_idx)


def combine(y: torch.Tensor, topk_weights: torch.Tensor, plan: DispatchPlan, group=None) -> torch.Tensor:
    """Inverse of dispatch for the experts' outputs y (expert-major), followed by the top-k weighted sum per token
    (fp32 accumulate in k order, one cast)."""
    tokens, topk = topk_weights.shape
    if plan.regroup_idx is not None:
        src_major = _gather_rows(y, plan.regroup_inv)            # a gather; the scatter form is several times slower
        back = y.new_empty(int(sum(plan.send_splits)), y.shape[1])
        dist.all_to_all_single(back, src_major, plan.send_splits, plan.recv_splits, group=group)
    else:
        back = y
    pos = plan.pos
    if back.is_cuda:
        return _combine_cuda(back, pos, topk_weights, tokens, topk)
    return (back[pos].reshape(tokens, topk, -1).float() * topk_weights.unsqueeze(-1).float()).sum(1).to(y.dtype)


def _combine_cuda(back, pos, topk_weights, tokens, topk):
    import ctypes
    from . import _lib
    back = back if back.stride(1) == 1 else back.contiguous()
    w = topk_weights.to(torch.float32).contiguous()
    out = back.new_empty(tokens, back.shape[1])
    with torch.cuda.device(back.device):
        rc = _lib.lib.tb_moe_combine(ctypes.c_void_p(back.data_ptr()), back.stride(0), ctypes.c_void_p(pos.data_ptr()),
                                     ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(out.data_ptr()), out.stride(0),
                                     tokens, topk, back.shape[1], _lib.DTYPE_CODE[back.dtype],
                                     _lib.current_stream_ptr(back.device))
    _lib.check(rc, "tb_moe_combine")
    return out


def swiglu(h: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for h = [gate | up] (fp32 math, one cast); the activation sits between the two projections and is
    outside the GEMM contract. One streaming CUDA kernel on the GPU; the CPU form serves the gloo tests."""
    if not h.is_cuda:
        gate, up = h.chunk(2, dim=-1)
        return torch.nn.functional.silu(gate.float()).mul_(up.float()).to(h.dtype)
    import ctypes
    from . import _lib
    h = h if h.stride(1) == 1 else h.contiguous()
    ffn = h.shape[1] // 2
    out = h.new_empty(h.shape[0], ffn)
    with torch.cuda.device(h.device):
        rc = _lib.lib.tb_swiglu(ctypes.c_void_p(h.data_ptr()), h.stride(0), ctypes.c_void_p(out.data_ptr()), out.stride(0),
                                h.shape[0], ffn, _lib.DTYPE_CODE[h.dtype], _lib.current_stream_ptr(h.device))
    _lib.check(rc, "tb_swiglu")
    return out


def _gate_up_swiglu(grouped_fn, rows, w1, group_offsets, row_index=None):
    """silu(rows @ gate.T) * (rows @ up.T) for w1 = [gate | up]: on the GPU with this library's grouped GEMM the activation
    runs inside the GEMM's epilogue when the shape allows it (ffn a multiple of 128, more than 128 rows); otherwise GEMM,
    then `swiglu`. ``row_index`` (this library's grouped GEMM only): the rows are picked from ``rows`` by index inside the
    kernel."""
    from .matmul import grouped_matmul
    kw = {} if row_index is None else {"row_index": row_index}
    n_rows = rows.shape[0] if row_index is None else row_index.numel()
    if grouped_fn is grouped_matmul and rows.is_cuda and (w1.shape[1] // 2) % 128 == 0 and n_rows > 128:
        return grouped_fn(rows, w1, group_offsets, swiglu=True, **kw)
    return swiglu(grouped_fn(rows, w1, group_offsets, **kw))


class ExpertParallelMoE:
    """Expert-parallel MoE feed-forward: gate/up projection, SwiGLU, down projection, with all-to-all token dispatch.

    w1: (experts_per_rank, 2*ffn, hidden) and w2: (experts_per_rank, hidden, ffn) hold this rank's experts, K-contiguous.
    """

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, num_experts: int, group=None, grouped_fn: Optional[Callable] = None,
                 expert_place: Optional[torch.Tensor] = None):
        self.w1, self.w2, self.num_experts, self.group = w1, w2, num_experts, group
        self.expert_place = expert_place        # expert id -> position in the layout order; w1 / w2 follow that order
        if grouped_fn is None:
            from .matmul import grouped_matmul as grouped_fn
        self.grouped_fn = grouped_fn

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor):
        plan = plan_dispatch(topk_ids, self.num_experts, self.group, self.expert_place)
        rows = dispatch(x, topk_ids.shape[1], plan, self.group)
        y = self.grouped_fn(_gate_up_swiglu(self.grouped_fn, rows, self.w1, plan.group_offsets), self.w2, plan.group_offsets)
        return combine(y, topk_weights, plan, self.group), plan


# ---------------------------------------------------------------------------------------------- peer-memory MoE path
@dataclass
class PeerDispatchPlan:
    """Where every (token, k) pair of this rank goes when rows are written straight into the owners' receive buffers.

    ``plan_peer_dispatch`` (torch index arithmetic, any device: the specification the CPU tests check) lists the rows in
    expert-sorted order; ``PeerMemoryMoE.plan`` (two CUDA kernels) lists them in pair order with ``src_token`` None
    (entry i is pair i, token i // topk) and leaves the order of the rows inside an expert unspecified."""
    src_token: Optional[torch.Tensor]   # int64 (n,)  token of the i-th row; None: entry i is the flattened pair i
    dest_rank: torch.Tensor      # int32 (n,)  rank that owns the row's expert
    dest_row: torch.Tensor       # int64 (n,)  row in that rank's receive buffer
    pair_rank: torch.Tensor      # int32 (tokens*topk,)  the same, indexed by the flattened (token, k) pair
    pair_row: torch.Tensor       # int64 (tokens*topk,)
    group_offsets: torch.Tensor  # int32 (experts_per_rank + 1,) row offsets of this rank's experts in its receive buffer
    row_token: Optional[torch.Tensor] = None   # int32 (capacity,) single rank only: source token of every row


def plan_peer_dispatch(topk_ids: torch.Tensor, counts_all: torch.Tensor, rank: int,
                       capacity: Optional[int] = None) -> PeerDispatchPlan:
    """Pure index arithmetic on the device (no host synchronisation).

    ``capacity``: rows of every rank's receive buffer. Rows routed beyond it are dropped by the dispatch kernel (and
    counted); the group offsets returned here are clamped to it, so the grouped GEMMs and the combine step never reach
    past the buffers either.

    counts_all: int64 (world, num_experts), counts_all[r, e] = pairs of rank r routed to expert e (every rank holds the
    same matrix after an all-gather of its own bincount). Expert e lives on rank e // experts_per_rank; inside that
    rank's receive buffer the experts follow each other, and inside an expert the source ranks follow each other, each
    source's rows in its own stable expert-sorted order.
    """
    world, num_experts = counts_all.shape
    epr = num_experts // world
    flat = topk_ids.reshape(-1).to(torch.int64)
    n = flat.numel()
    sort_idx = torch.argsort(flat, stable=True)
    e_sorted = flat[sort_idx]
    totals = counts_all.sum(0)                                              # rows per expert over all sources
    per_owner = totals.view(world, epr)
    owner_off = (per_owner.cumsum(1) - per_owner).reshape(-1)               # start of expert e inside its owner's buffer
    dest_base = owner_off + counts_all[:rank].sum(0)                        # + rows of lower-ranked sources
    mine = counts_all[rank]
    my_start = mine.cumsum(0) - mine                                        # start of expert e in my sorted list
    i = torch.arange(n, device=flat.device)
    dest_row = dest_base[e_sorted] + (i - my_start[e_sorted])
    dest_rank = (e_sorted // epr).to(torch.int32)
    pair_row = torch.empty_like(dest_row)
    pair_row[sort_idx] = dest_row
    pair_rank = torch.empty_like(dest_rank)
    pair_rank[sort_idx] = dest_rank
    group_offsets = torch.zeros(epr + 1, dtype=torch.int32, device=flat.device)
    ends = per_owner[rank].cumsum(0)
    if capacity is not None:
        ends = ends.clamp(max=int(capacity))
    group_offsets[1:] = ends.to(torch.int32)
    topk = topk_ids.shape[1]
    return PeerDispatchPlan(sort_idx // topk, dest_rank, dest_row, pair_rank, pair_row, group_offsets)


class PeerMemoryMoE:
    """Expert-parallel MoE feed-forward whose token exchange runs over peer-mapped memory instead of collectives.

    Every rank allocates a receive buffer and an output buffer of ``capacity`` rows in symmetric memory. The dispatch plan
    is two small kernels (per-expert counts; row of every (token, k) pair in its owner's buffer), dispatch is ONE kernel
    that writes each routed row into its owner's receive buffer over NVLink, already in the order the grouped GEMM wants;
    combine is ONE kernel that reads the experts' outputs from the owners' buffers and forms the top-k weighted sum. Two
    symmetric-memory barriers per call order the phases; the only collective is an all-gather of the per-expert counts
    (world x experts integers), and nothing synchronises with the host. Rows routed beyond ``capacity`` are dropped and
    counted in ``overflow``; the tokens they belong to lose that expert's contribution.

    With one rank (no process group) the same kernels run on ordinary device buffers, without barriers or collectives.
    """

    def __init__(self, w1: torch.Tensor, w2: torch.Tensor, num_experts: int, capacity: int, group=None,
                 expert_place: Optional[torch.Tensor] = None, gather_rows: bool = False):
        import ctypes
        self.w1, self.w2, self.num_experts, self.group = w1, w2, num_experts, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert num_experts % self.world == 0, "experts must divide evenly over the ranks"
        hidden = w1.shape[2]
        self.capacity, self.hidden = int(capacity), hidden
        dev = w1.device
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            pg = group if group is not None else dist.group.WORLD
            self.recv = symm_mem.empty(self.capacity, hidden, dtype=w1.dtype, device=dev)
            self.recv_h = symm_mem.rendezvous(self.recv, group=pg)
            self.y = symm_mem.empty(self.capacity, hidden, dtype=w1.dtype, device=dev)
            self.y_h = symm_mem.rendezvous(self.y, group=pg)
            recv_ptrs, y_ptrs = self.recv_h.buffer_ptrs, self.y_h.buffer_ptrs
        else:
            self.recv = torch.empty(self.capacity, hidden, dtype=w1.dtype, device=dev)
            self.y = torch.empty(self.capacity, hidden, dtype=w1.dtype, device=dev)
            self.recv_h = self.y_h = None
            recv_ptrs, y_ptrs = [self.recv.data_ptr()], [self.y.data_ptr()]
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)   # rows dropped because capacity was too small
        self._recv_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in recv_ptrs])
        self._y_ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in y_ptrs])
        # plan state: this rank's counts, every rank's counts, the per-expert cursor, row offsets of the local experts
        self._counts = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self._counts_all = torch.zeros(self.world, num_experts, dtype=torch.int32, device=dev)
        self._cursor = torch.zeros(num_experts, dtype=torch.int32, device=dev)
        self._pairs = {}       # n_pairs -> (pair_rank int32, pair_row int64)
        # One rank, on request: the gate/up GEMM picks the tokens' rows straight from x by index (gather-mode TMA copies, no
        # dispatch copy, no receive buffer). Measured on B200: a gather-mode copy moves four 128-byte rows and the copy
        # unit retires one about every 90 clocks, 5-6 bytes per clock and SM where a tensor-bound tile needs 32, so the
        # projection runs three times slower than on rows copied into place first (0.28 ms for 131072 x 4096 bf16 rows);
        # it pays only where the grouped GEMM is not bound by its operand rate. Off by default.
        self._gather_rows = bool(gather_rows) and self.world == 1 and w1.element_size() == 2 and hidden % 8 == 0
        self._row_token = None
        # expert id -> position in the layout order (w1 / w2 hold this rank's experts in that order); None = identity
        self._place = None if expert_place is None else expert_place.to(device=dev, dtype=torch.int32).contiguous()
        if self._place is not None:
            assert self._place.numel() == num_experts and sorted(self._place.tolist()) == list(range(num_experts))

    def plan(self, topk_ids: torch.Tensor) -> PeerDispatchPlan:
        """Device-side dispatch plan of ``topk_ids`` (tokens, topk): no sort, no host synchronisation."""
        import ctypes
        from . import _lib
        ids = topk_ids if topk_ids.is_contiguous() else topk_ids.contiguous()
        assert ids.dtype in (torch.int32, torch.int64), "expert ids must be int32 or int64"
        n = ids.numel()
        if n not in self._pairs:
            self._pairs[n] = (torch.empty(n, dtype=torch.int32, device=ids.device),
                              torch.empty(n, dtype=torch.int64, device=ids.device))
        pair_rank, pair_row = self._pairs[n]
        group_offsets = torch.empty(self.num_experts // self.world + 1, dtype=torch.int32, device=ids.device)
        row_token = None
        if self._gather_rows:
            if self._row_token is None:
                self._row_token = torch.full((self.capacity,), -1, dtype=torch.int32, device=ids.device)
            row_token = self._row_token
        stream = _lib.current_stream_ptr(ids.device)
        is64 = int(ids.dtype == torch.int64)
        with torch.cuda.device(ids.device):
            place = ctypes.c_void_p(self._place.data_ptr() if self._place is not None else 0)
            rc = _lib.lib.tb_moe_count(ctypes.c_void_p(ids.data_ptr()), is64, n, self.num_experts, place,
                                       ctypes.c_void_p(self._counts.data_ptr()), stream)
            _lib.check(rc, "tb_moe_count")
            if self.world > 1:
                dist.all_gather_into_tensor(self._counts_all.view(-1), self._counts, group=self.group)
                counts_all = self._counts_all
            else:
                counts_all = self._counts
            rc = _lib.lib.tb_moe_plan(ctypes.c_void_p(ids.data_ptr()), is64, n, self.num_experts, place, self.world, self.rank,
                                      ctypes.c_void_p(counts_all.data_ptr()), ctypes.c_void_p(self._cursor.data_ptr()),
                                      self.capacity, ctypes.c_void_p(pair_rank.data_ptr()), ctypes.c_void_p(pair_row.data_ptr()),
                                      ctypes.c_void_p(group_offsets.data_ptr()),
                                      ctypes.c_void_p(row_token.data_ptr() if row_token is not None else 0),
                                      int(topk_ids.shape[1]), stream)
            _lib.check(rc, "tb_moe_plan")
        return PeerDispatchPlan(None, pair_rank, pair_row, pair_rank, pair_row, group_offsets, row_token)

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, phase_events=None):
        """``phase_events``: a list that receives (name, torch.cuda.Event) after each phase (plan, dispatch, gate_up, down,
        combine) for a timing breakdown; each closes with the barrier that follows it, if any."""
        import ctypes
        from . import _lib
        from .matmul import grouped_matmul
        tokens, topk = topk_ids.shape

        def mark(name):
            if phase_events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                phase_events.append((name, ev))

        mark("start")
        plan = self.plan(topk_ids)
        mark("plan")
        stream = _lib.current_stream_ptr(x.device)
        code = _lib.DTYPE_CODE[x.dtype]
        x = x if x.stride(1) == 1 else x.contiguous()
        gather = plan.row_token is not None and (x.stride(0) * x.element_size()) % 16 == 0 and x.data_ptr() % 16 == 0
        if gather:
            mark("dispatch")
            act = _gate_up_swiglu(grouped_matmul, x, self.w1, plan.group_offsets, row_index=plan.row_token)
        else:
            with torch.cuda.device(x.device):
                rc = _lib.lib.tb_moe_dispatch_peers(ctypes.c_void_p(x.data_ptr()), x.stride(0), ctypes.c_void_p(0),
                                                    ctypes.c_void_p(plan.pair_rank.data_ptr()),
                                                    ctypes.c_void_p(plan.pair_row.data_ptr()), self._recv_ptrs, self.world,
                                                    self.recv.stride(0), self.capacity,
                                                    ctypes.c_void_p(self.overflow.data_ptr()), tokens * topk, self.hidden,
                                                    code, topk, stream)
            _lib.check(rc, "tb_moe_dispatch_peers")
            if self.recv_h is not None:
                self.recv_h.barrier(channel=0)              # every rank's rows have landed in every receive buffer
            mark("dispatch")
            act = _gate_up_swiglu(grouped_matmul, self.recv, self.w1, plan.group_offsets)
        mark("gate_up")
        grouped_matmul(act, self.w2, plan.group_offsets, out=self.y)
        if self.y_h is not None:
            self.y_h.barrier(channel=0)                     # every rank's expert outputs are complete
        mark("down")
        w = topk_weights.to(torch.float32).contiguous()
        out = x.new_empty(tokens, self.hidden)
        with torch.cuda.device(x.device):
            rc = _lib.lib.tb_moe_combine_peers(self._y_ptrs, self.world, self.y.stride(0),
                                               ctypes.c_void_p(plan.pair_rank.data_ptr()),
                                               ctypes.c_void_p(plan.pair_row.data_ptr()), ctypes.c_void_p(w.data_ptr()),
                                               ctypes.c_void_p(out.data_ptr()), out.stride(0), tokens, topk, self.hidden,
                                               code, self.capacity, stream)
        _lib.check(rc, "tb_moe_combine_peers")
        mark("combine")
        return out, plan
