"""Grouped (MoE) GEMM against the CPU oracle's per-group loop; tolerance as for the dense bf16 GEMM (rtol 1e-2 + 1e-2 rms)."""
import pytest
import torch

import tritonblas_b200 as tb
from oracle import gemm_oracle

pytestmark = pytest.mark.gpu


def _case(counts, n, k, dtype=torch.bfloat16, seed=0):
    g = torch.Generator().manual_seed(seed)
    rows = sum(counts)
    x = torch.randn(rows, k, generator=g).to(dtype).cuda()
    w = (torch.randn(len(counts), n, k, generator=g) * 0.05).to(dtype).cuda()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0).tolist()), dtype=torch.int32).cuda()
    return x, w, offs


def _check(y, x, w, offs, what):
    ref = gemm_oracle.grouped_gemm_ref(x, w.transpose(1, 2), offs.cpu(), torch.float32)
    got = y.float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs()
    bad = err > 1e-2 * ref.abs() + 1e-2 * max(rms, 1e-30)
    assert torch.isfinite(got).all(), what
    assert not bad.any(), f"{what}: {int(bad.sum())} off, max err {err.max().item():.4g}, rms {rms:.4g}, first {bad.nonzero()[0].tolist()}"


@pytest.mark.parametrize("counts", [[128, 128], [256, 0, 300, 1, 77], [5, 9, 1000, 130, 0, 0, 513], [0, 0, 64], [1] * 40])
@pytest.mark.parametrize("n,k", [(256, 256), (384, 512), (200, 320)])
def test_grouped_matches_oracle(counts, n, k):
    x, w, offs = _case(counts, n, k, seed=len(counts) + n)
    y = torch.full((x.shape[0], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    tb.grouped_matmul(x, w, offs, out=y)
    _check(y, x, w, offs, f"grouped {counts} n={n} k={k}")
    assert tb.device_status() == 0


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("counts", [[256, 0, 300, 1, 77], [5, 9, 1000, 130, 0, 0, 513]])
@pytest.mark.parametrize("n,k", [(512, 256), (768, 512), (1100, 320)])
def test_grouped_wide_tiles(counts, n, k, pair):
    """Wide tiles (two accumulators per work tile) in grouped mode, with group widths that end on a tile, in the first
    half of one and in the second half of one."""
    x, w, offs = _case(counts, n, k, seed=len(counts) + n)
    y = torch.full((x.shape[0], n), float("nan"), dtype=torch.bfloat16, device="cuda")
    bf = torch.bfloat16
    sel = tb.OrigamiMatmulSelector(x.shape[0], n, k, bf, bf, bf, torch.device("cuda", 0))
    sel.override(cta_pair=pair, block_n=256, n_halves=2)
    tb.grouped_matmul(x, w, offs, out=y, selector=sel)
    _check(y, x, w, offs, f"grouped wide {counts} n={n} k={k} pair={pair}")
    assert tb.device_status() == 0


@pytest.mark.parametrize("counts", [[256, 0, 300, 1, 77], [5, 9, 1000, 130, 0, 0, 513], [128] * 8])
@pytest.mark.parametrize("ffn,k", [(256, 256), (384, 512), (1536, 320), (128, 128)])
def test_grouped_gate_up_with_fused_swiglu(counts, ffn, k):
    """swiglu=True: w = [gate | up]; the epilogue applies silu(gate) * up to the fp32 accumulators. Reference: the same
    product in fp32 on the CPU (oracle grouped GEMM on both halves), activation in fp32, one cast."""
    x, w, offs = _case(counts, 2 * ffn, k, seed=ffn + k)
    y = torch.full((x.shape[0], ffn), float("nan"), dtype=torch.bfloat16, device="cuda")
    tb.grouped_matmul(x, w, offs, out=y, swiglu=True)
    h = gemm_oracle.grouped_gemm_ref(x, w.transpose(1, 2), offs.cpu(), torch.float32)
    ref = torch.nn.functional.silu(h[:, :ffn]) * h[:, ffn:]
    got = y.float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs()
    assert torch.isfinite(got).all()
    assert not (err > 1e-2 * ref.abs() + 1e-2 * max(rms, 1e-30)).any(), f"max err {err.max().item():.4g} rms {rms:.4g}"
    assert tb.device_status() == 0


@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_dynamic_schedule_is_bit_identical(swiglu):
    counts = [5, 9, 1000, 130, 0, 0, 513, 2048, 77]
    x, w, offs = _case(counts, 512, 384, seed=5)
    ref = tb.grouped_matmul(x, w, offs, swiglu=swiglu)
    for _ in range(3):
        got = tb.grouped_matmul(x, w, offs, swiglu=swiglu, work_stealing=True)
        assert torch.equal(got, ref)
    assert tb.device_status() == 0


def test_grouped_moe_projection_shapes():
    """BASELINE config 5 at full size: 64 experts, top-8 of 16384 tokens (131072 rows), Zipf(1.1)-skewed counts, hidden
    4096, ffn 1536; gate/up (N = 3072) and down (N = 4096) projections, 48 sampled rows checked per projection."""
    g = torch.Generator().manual_seed(7)
    E, tokens, topk = 64, 16384, 8
    p = (torch.arange(1, E + 1, dtype=torch.float64) ** -1.1)
    p = (p / p.sum())[torch.randperm(E, generator=g)]
    choice = torch.multinomial(p.expand(tokens, E), topk, replacement=False, generator=g)
    counts = torch.bincount(choice.flatten(), minlength=E).tolist()
    gd = torch.Generator(device="cuda").manual_seed(11)
    for n, k in ((3072, 4096), (4096, 1536)):
        # generated on the device: the host copy of these operands would be several GB of fp32
        x = torch.randn(sum(counts), k, device="cuda", generator=gd).to(torch.bfloat16)
        w = (torch.randn(E, n, k, device="cuda", generator=gd) * 0.05).to(torch.bfloat16)
        offs = torch.tensor([0] + torch.tensor(counts).cumsum(0).tolist(), dtype=torch.int32, device="cuda")
        y = tb.grouped_matmul(x, w, offs)
        rows = torch.randint(0, x.shape[0], (48,), generator=g)
        # oracle on the sampled rows only: find each row's expert from the offsets
        expert = torch.bucketize(rows, offs.cpu().long()[1:], right=True)
        for r, e in zip(rows.tolist(), expert.tolist()):
            ref = x[r].float().cpu() @ w[e].float().cpu().T
            got = y[r].float().cpu()
            rms = ref.pow(2).mean().sqrt()
            assert ((got - ref).abs() <= 1e-2 * ref.abs() + 1e-2 * rms).all(), (n, k, r, e)
    assert tb.device_status() == 0


def test_swiglu_and_combine_kernels_match_fp32_formulas():
    from tritonblas_b200 import distributed as tbd
    g = torch.Generator().manual_seed(3)
    h = torch.randn(333, 2 * 256, generator=g).to(torch.bfloat16).cuda()
    got = tbd.swiglu(h).float().cpu()
    gate, up = h.float().cpu().chunk(2, dim=-1)
    ref = torch.nn.functional.silu(gate) * up
    assert torch.allclose(got, ref, rtol=1e-2, atol=1e-2)
    tokens, topk, hidden, E = 50, 4, 512, 8
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(tokens)]).cuda()
    plan = tbd.plan_dispatch(ids, E)
    x = torch.randn(tokens, hidden, generator=g).to(torch.bfloat16).cuda()
    rows = tbd.dispatch(x, topk, plan)                       # expert-major copies of the token rows
    w = torch.rand(tokens, topk, generator=g).cuda()
    out = tbd.combine(rows, w, plan).float().cpu()
    ref = x.float().cpu() * w.sum(1, keepdim=True).cpu()     # every copy is the token itself
    assert torch.allclose(out, ref, rtol=1e-2, atol=1e-2)
    assert tb.device_status() == 0


def test_row_gather_kernel_matches_index_select():
    from tritonblas_b200 import distributed as tbd
    g = torch.Generator().manual_seed(9)
    for rows, hidden in ((1, 8), (333, 520), (4096, 4096)):
        x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).cuda()
        idx = torch.randint(0, rows, (3 * rows + 5,), generator=g).cuda()
        assert torch.equal(tbd._gather_rows(x, idx), x.index_select(0, idx))
        view = x[:, : hidden - (hidden % 16 or 8)] if hidden > 8 else x          # a row-strided view keeps the kernel path
        assert torch.equal(tbd._gather_rows(view, idx), view.index_select(0, idx))
    assert tb.device_status() == 0


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("counts", [[256, 0, 300, 1, 77], [5, 9, 1000, 130, 0, 0, 513], [128] * 8, [3000]])
@pytest.mark.parametrize("n,k", [(256, 256), (384, 520), (200, 1024)])
def test_grouped_with_rows_gathered_by_index(counts, n, k, pair):
    """row_index: grouped row r is row row_index[r] of x (tokens repeat; order arbitrary; a negative entry is a zero row).
    The kernel's producer loads the rows with gather-mode TMA copies; compared with the oracle on the explicitly gathered matrix. k = 520 ends
    inside a 64-element stage."""
    tokens = 700
    g = torch.Generator().manual_seed(sum(counts) + n + k)
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(len(counts), n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    rows = sum(counts)
    idx = torch.randint(0, tokens, (rows,), generator=g).to(torch.int32)
    idx[::97] = -1
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0).tolist()), dtype=torch.int32).cuda()
    gathered = x[idx.clamp(min=0).long().cuda()] * (idx >= 0).cuda().unsqueeze(1).to(x.dtype)
    y = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    bf = torch.bfloat16
    sel = tb.OrigamiMatmulSelector(rows, n, k, bf, bf, bf, torch.device("cuda", 0), max_halves=1)
    sel.override(cta_pair=pair, block_n=128 if n < 256 else 256)
    for ws in (False, True):
        y.fill_(float("nan"))
        tb.grouped_matmul(x, w, offs, out=y, selector=sel, row_index=idx.cuda(), work_stealing=ws)
        _check(y, gathered, w, offs, f"gathered rows {counts} n={n} k={k} pair={pair} ws={ws}")
    assert tb.device_status() == 0


def test_grouped_gate_up_swiglu_with_rows_gathered_by_index():
    counts, ffn, k, tokens = [256, 0, 300, 1, 77, 1200], 256, 512, 500
    g = torch.Generator().manual_seed(3)
    x = torch.randn(tokens, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(len(counts), 2 * ffn, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    rows = sum(counts)
    idx = torch.randint(0, tokens, (rows,), generator=g).to(torch.int32).cuda()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0).tolist()), dtype=torch.int32).cuda()
    direct = tb.grouped_matmul(x[idx.long()].contiguous(), w, offs, swiglu=True)
    fused = tb.grouped_matmul(x, w, offs, swiglu=True, row_index=idx)
    assert torch.equal(direct, fused)        # same tiles, same arithmetic: only the way A reaches shared memory differs
    assert tb.device_status() == 0
