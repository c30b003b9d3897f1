"""GPU parity of the dense GEMM family against the CPU oracle, through the public API (which calls the C ABI).

Tolerance (stated by the task): rtol 1e-2 for fp16/bf16 outputs against the fp32-accumulate product; an absolute term of
1e-2 * rms(reference) covers elements that cancel to near zero.
"""
import pytest
import torch

import tritonblas_b200 as tb
from tests._util import assert_close_to_oracle, make_operands
from tests.conftest import EDGE_CASE_DIMS, STANDARD_DIMS

pytestmark = pytest.mark.gpu

LAYOUTS = [("T", "T"), ("T", "N"), ("N", "T"), ("N", "N")]


def _selector(m, n, k, dt, out_dt=None, streamk=False, **override):
    s = tb.OrigamiMatmulSelector(m, n, k, dt, dt, out_dt or dt, torch.device("cuda", 0), streamk=streamk)
    if override:
        s.override(**override)
    return s


@pytest.fixture(autouse=True)
def _no_device_failure():
    yield
    assert tb.device_status() == 0


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("ta,tb_", LAYOUTS)
def test_fp16_1024_all_layouts(ta, tb_, pair):
    """BASELINE config 1: fp16 1024^3, N(0,1) inputs, fp32 accumulate, fp16 out, every operand layout."""
    a, b = make_operands(1024, 1024, 1024, torch.float16, ta, tb_)
    c = torch.empty(1024, 1024, dtype=torch.float16, device="cuda")
    sel = _selector(1024, 1024, 1024, torch.float16, cta_pair=pair, block_n=128)
    tb.matmul_lt(a, b, c, sel, None)
    assert_close_to_oracle(c, a, b, what=f"fp16 1024 {ta}{tb_} pair={pair}")


@pytest.mark.parametrize("pair,bn", [(1, 32), (1, 64), (1, 128), (1, 256), (2, 64), (2, 128), (2, 256)])
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_tile_shapes(dt, pair, bn):
    m, n, k = 640, 768, 512
    a, b = make_operands(m, n, k, dt, "T", "T", seed=3)
    c = torch.empty(m, n, dtype=dt, device="cuda")
    tb.matmul_lt(a, b, c, _selector(m, n, k, dt, cta_pair=pair, block_n=bn), None)
    assert_close_to_oracle(c, a, b, what=f"{dt} pair={pair} bn={bn}")


@pytest.mark.parametrize("pair,bn", [(1, 128), (1, 256), (2, 128), (2, 256)])
@pytest.mark.parametrize("ta,tb_", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(512, 1024, 512), (300, 700, 264), (1024, 520, 1024), (256, 4104, 512)])
def test_wide_tiles(m, n, k, ta, tb_, pair, bn):
    """n_halves = 2: a work tile is two accumulators side by side that share every A stage. Covers widths that end
    inside the first half, inside the second half and exactly on a tile, for every operand layout."""
    a, b = make_operands(m, n, k, torch.bfloat16, ta, tb_, seed=11)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    tb.matmul_lt(a, b, c, _selector(m, n, k, torch.bfloat16, cta_pair=pair, block_n=bn, n_halves=2), None)
    assert_close_to_oracle(c, a, b, what=f"wide {(m, n, k)} {ta}{tb_} pair={pair} bn={bn}")


def test_wide_tiles_with_bias_and_fp32_output():
    m, n, k = 384, 1536, 512
    a, b = make_operands(m, n, k, torch.float16, "T", "T", seed=12)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(4)).to(torch.float16).cuda()
    for out_dt in (torch.float16, torch.float32):
        c = torch.empty(m, n, dtype=out_dt, device="cuda")
        sel = _selector(m, n, k, torch.float16, out_dt=out_dt, block_n=256, n_halves=2)
        tb.persistent_matmul_lt(a, b, c, sel, None, bias=bias)
        assert_close_to_oracle(c, a, b, bias=bias, what=f"wide bias out={out_dt}")


def test_selector_takes_wide_tiles_for_large_k_only():
    dev = torch.device("cuda", 0)
    bf = torch.bfloat16
    assert tb.OrigamiMatmulSelector(8192, 8192, 8192, bf, bf, bf, dev).config_for(False, False).n_halves == 2
    assert tb.OrigamiMatmulSelector(8192, 8192, 512, bf, bf, bf, dev).config_for(False, False).n_halves == 1
    assert tb.OrigamiMatmulSelector(8192, 8192, 8192, bf, bf, bf, dev, streamk=True).config_for(False, False).n_halves == 1


@pytest.mark.parametrize("m,n,k", STANDARD_DIMS + EDGE_CASE_DIMS)
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_matmul_default_selector(m, n, k, dt):
    """tritonblas.matmul with the library's own choice of configuration, row-major A and B (N-contiguous B)."""
    a, b = make_operands(m, n, k, dt, "T", "N", seed=42)
    c = tb.matmul(a, b)
    assert c.dtype == dt and tuple(c.shape) == (m, n)
    assert_close_to_oracle(c, a, b, what=f"{(m, n, k)} {dt}")


@pytest.mark.parametrize("ta,tb_", LAYOUTS)
@pytest.mark.parametrize("m,n,k", [(257, 129, 200), (15, 17, 512), (130, 260, 72), (4864 // 8, 8192 // 8, 4160 // 8)])
def test_ragged_shapes_all_layouts(m, n, k, ta, tb_):
    a, b = make_operands(m, n, k, torch.bfloat16, ta, tb_, seed=9)
    c = tb.matmul(a, b)
    assert_close_to_oracle(c, a, b, what=f"{(m, n, k)} {ta}{tb_}")


@pytest.mark.parametrize("pair,bn,nh", [(1, 128, 1), (2, 256, 1), (2, 256, 2), (1, 256, 2), (2, 64, 1)])
@pytest.mark.parametrize("m,n,k", [(2048, 4096, 512), (1000, 3000, 264), (256, 256, 1024)])
def test_work_stealing_schedule_matches_oracle(m, n, k, pair, bn, nh):
    """work_stealing=True: tiles after each program's first come from a device counter. Three launches in a row share the
    counter words, which the kernel leaves zeroed every time; results equal the static schedule's bit for bit (the same
    tiles are computed the same way, only by different programs)."""
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=31)
    sel = _selector(m, n, k, torch.bfloat16, cta_pair=pair, block_n=bn, n_halves=nh)
    cfg = tb.matmul_preamble(sel)
    ref = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_lt(a, b, ref, sel, cfg)
    assert_close_to_oracle(ref, a, b, what=f"static {(m, n, k)} pair={pair} bn={bn} nh={nh}")
    for rep in range(3):
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        tb.matmul_lt(a, b, c, sel, cfg, work_stealing=True)
        assert torch.equal(c, ref), f"launch {rep}"
        assert int(cfg.tile_counter[:2].abs().sum()) == 0


def test_work_stealing_through_matmul_and_addmm():
    m, n, k = 1536, 2048, 1024
    a, b = make_operands(m, n, k, torch.float16, "T", "N", seed=32)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(5)).to(torch.float16).cuda()
    for _ in range(2):
        c = tb.matmul(a, b, work_stealing=True)
        assert_close_to_oracle(c, a, b, what="matmul work_stealing")
        d = tb.addmm(bias, a, b, work_stealing=True)
        assert_close_to_oracle(d, a, b, bias=bias, what="addmm work_stealing")


@pytest.mark.parametrize("ta,tb_", LAYOUTS)
def test_large_unaligned_operands_take_the_tensor_core_path(ta, tb_):
    """K and N not multiples of 8: the operands' pitches are not 16-byte aligned, so the host re-pitches them (one copy
    each) instead of leaving a product this size to the CUDA-core kernel; results still match the oracle."""
    m, n, k = 1000, 1001, 1027
    a, b = make_operands(m, n, k, torch.bfloat16, ta, tb_, seed=21)
    c = tb.matmul(a, b)
    assert_close_to_oracle(c, a, b, what=f"unaligned {ta}{tb_}")


@pytest.mark.parametrize("m,n,k", [(300, 200, 100), (512, 768, 256), (64, 96, 0)])
def test_output_fan_out_to_further_buffers(m, n, k):
    """c_copies: every tile also goes to further buffers laid out like C (on several GPUs: the peers' gathered C). Checked on
    one GPU with local buffers, for operands TMA can address and for K % 8 != 0, which runs on the CUDA-core kernel; K = 0
    leaves bias only."""
    a, b = make_operands(m, n, max(k, 8), torch.bfloat16, "T", "T", seed=17)
    a, b = a[:, :k].contiguous(), b[:k].T.contiguous().T          # K-contiguous with pitch K: unaligned when K % 8 != 0
    bias = torch.randn(n, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    copies = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    sel = tb.OrigamiMatmulSelector(m, n, max(k, 1), torch.bfloat16, torch.bfloat16, torch.bfloat16, torch.device("cuda", 0),
                                   max_halves=1)
    tb.persistent_matmul_lt(a, b, c, sel, None, bias=bias, c_copies=[t.data_ptr() for t in copies])
    assert_close_to_oracle(c, a, b, bias=bias, what=f"fan-out {(m, n, k)}")
    for t in copies:
        assert torch.equal(t, c)


@pytest.mark.parametrize("fraction", [0.3, 0.5, 1.0])
@pytest.mark.parametrize("m,n,k,pair,bn,nh", [(2048, 4096, 512, 2, 256, 1), (1000, 3000, 264, 1, 128, 1), (2048, 4096, 512, 2, 256, 2),
                                              (520, 776, 128, 2, 64, 1)])
def test_output_fan_out_with_the_tail_tiles_sent_after_the_launch(m, n, k, pair, bn, nh, fraction):
    """c_copies_tail_fraction: the epilogue sends only the launch's first tiles to the further buffers; a copy kernel on a
    side stream sends the rest in the kernel's own tile order. Afterwards every buffer holds the whole product (checked on
    one GPU with local buffers; ragged right and bottom edges included)."""
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=19)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    copies = [torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    sel = _selector(m, n, k, torch.bfloat16, cta_pair=pair, block_n=bn, n_halves=nh)
    side = torch.cuda.Stream()
    for ws in (False, True):       # static and dynamic tile schedule (the tile index decides who sends a tile, not the program)
        c.fill_(float("nan"))
        for t in copies:
            t.fill_(float("nan"))
        tb.persistent_matmul_lt(a, b, c, sel, None, c_copies=[t.data_ptr() for t in copies], c_copies_tail_stream=side,
                                c_copies_tail_fraction=fraction, work_stealing=ws)
        torch.cuda.current_stream().wait_stream(side)
        assert_close_to_oracle(c, a, b, what=f"tail fan-out {(m, n, k)} ws={ws}")
        for t in copies:
            assert torch.equal(t, c)


@pytest.mark.parametrize("pair", [1, 2])
def test_strided_output_and_out_argument(pair):
    m, n, k = 300, 200, 256
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T")
    big = torch.zeros(m, n + 56, dtype=torch.bfloat16, device="cuda")
    c = big[:, 8:8 + n]
    tb.matmul_lt(a, b, c, _selector(m, n, k, torch.bfloat16, cta_pair=pair, block_n=64), None)
    assert_close_to_oracle(c, a, b)
    assert big[:, :8].abs().sum() == 0 and big[:, 8 + n:].abs().sum() == 0
    ct = torch.empty(n, m, dtype=torch.bfloat16, device="cuda").T  # column-major output
    assert tb.matmul(a, b, out=ct) is None
    assert_close_to_oracle(ct, a, b)


def test_fp32_output_from_bf16_inputs():
    m, n, k = 256, 384, 320
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T")
    c = torch.empty(m, n, dtype=torch.float32, device="cuda")
    tb.matmul_lt(a, b, c, _selector(m, n, k, torch.bfloat16, torch.float32), None)
    assert_close_to_oracle(c, a, b, rtol=1e-4)


@pytest.mark.parametrize("ta,tb_", LAYOUTS)
@pytest.mark.parametrize("allow_tf32", [True, False])
def test_fp32_inputs(ta, tb_, allow_tf32):
    """fp32 operands: tf32 tensor-core products when torch allows them (rtol 1e-2 like the 16-bit types; tf32 keeps 10
    mantissa bits), exact fp32 multiply-add otherwise (rtol 1e-5)."""
    m, n, k = 384, 320, 288
    a, b = make_operands(m, n, k, torch.float32, ta, tb_)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = allow_tf32
    try:
        c = tb.matmul(a, b)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert_close_to_oracle(c, a, b, rtol=1e-2 if allow_tf32 else 1e-5, what=f"fp32 {ta}{tb_} tf32={allow_tf32}")


def test_bf16_8192_cubed_sampled_rows():
    """BASELINE config 2a at full size: bf16 8192^3 TN, values N(0,1)*0.02; the oracle checks 48 sampled rows, and
    linearity (A@B with A doubled equals twice the product, exactly, since scaling by 2 is exact) covers the rest."""
    m = n = k = 8192
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=1, scale=0.02)
    c = tb.matmul(a, b)
    rows = torch.randint(0, m, (48,), generator=torch.Generator().manual_seed(5)).tolist() + [0, 127, 128, 255, 256, m - 1]
    assert_close_to_oracle(c, a, b, rows=rows, what="bf16 8192^3")
    c2 = tb.matmul(a * 2, b)
    assert torch.equal(c2, c * 2)


@pytest.mark.parametrize("pair", [1, 2])
@pytest.mark.parametrize("m,n,k,sk_grid", [(256, 512, 2048, 0), (384, 640, 4096, 37), (128, 256, 8192, 148),
                                           (1024, 1024, 1024, 50), (130, 100, 1000, 7), (16, 2048, 4096, 0)])
def test_streamk_matches_oracle_and_is_deterministic(m, n, k, sk_grid, pair):
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=11)
    sel = _selector(m, n, k, torch.bfloat16, streamk=True, cta_pair=pair, block_n=128)
    cfg = tb.matmul_preamble(sel)
    outs = []
    for _ in range(3):
        c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        if sk_grid:
            tb.streamk_matmul_lt(a, b, c, sel, cfg, sk_grid=sk_grid)
        else:
            tb.matmul_lt(a, b, c, sel, cfg, enable_streamk=True)
        outs.append(c)
    assert_close_to_oracle(outs[0], a, b, what=f"stream-K {(m, n, k)} grid={sk_grid} pair={pair}")
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])  # fix-up order is fixed


@pytest.mark.parametrize("trans_b", ["T", "N"])
@pytest.mark.parametrize("streamk", [False, True])
@pytest.mark.parametrize("m", [8, 128, 300])
def test_static_weights_are_read_before_the_previous_kernel_ends_and_nothing_else_is(m, streamk, trans_b):
    """static_b: the kernel may request b before the stream's previous kernel has finished. A chain of launches whose
    activations are each written by the kernel just before (the previous product, rescaled in place) must give the same
    values as the same chain without the promise; the weights alternate between two matrices."""
    n = k = 2048
    dt = torch.bfloat16
    w = [make_operands(n, n, k, dt, "T", trans_b, seed=70 + i, scale=0.03)[1] for i in range(2)]
    x0 = make_operands(m, n, k, dt, "T", "T", seed=3)[0]
    # single CTAs: the early request exists for them only (few rows: the weights are the tile's 128-row operand; more
    # rows: its column operand, K- or N-contiguous)
    sel = _selector(m, n, k, dt, streamk=streamk, cta_pair=1, block_n=128) if m > 64 else _selector(m, n, k, dt, streamk=streamk)
    cfg = tb.matmul_preamble(sel)

    def chain(static):
        x = x0.clone()
        outs = []
        for step in range(6):
            y = torch.empty(m, n, dtype=dt, device="cuda")
            tb.matmul_lt(x, w[step & 1], y, sel, cfg, enable_streamk=streamk, static_b=static)
            outs.append(y)
            x = y          # the next launch's activations are what this one is still writing
        return outs

    plain = chain(False)
    early = chain(True)
    assert_close_to_oracle(plain[0], x0, w[0], what="first link")
    for p_, e_ in zip(plain, early):
        assert torch.equal(p_, e_)


@pytest.mark.parametrize("m", [1, 16, 128])
def test_streamk_skinny_decode_shapes(m):
    """BASELINE config 2b: M in {1,16,128}, N=28672, K=8192, stream-K enabled; sampled columns checked."""
    n, k = 28672, 8192
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=2, scale=0.02)
    c = tb.matmul(a, b, enable_streamk=True)
    cols = torch.randint(0, n, (512,), generator=torch.Generator().manual_seed(6))
    cols = torch.cat([cols, torch.tensor([0, 127, 128, n - 1])]).to("cuda")
    assert_close_to_oracle(c[:, cols], a, b[:, cols], what=f"skinny m={m}")


def test_matmul_streamk_via_matmul_global_workspace():
    a, b = make_operands(512, 768, 1024, torch.float16, "T", "N")
    c1 = tb.matmul(a, b, enable_streamk=True, sk_grid=61)
    c2 = tb.matmul(a, b, enable_streamk=True, sk_grid=61)
    assert_close_to_oracle(c1, a, b)
    assert torch.equal(c1, c2)


@pytest.mark.parametrize("streamk", [False, True])
def test_addmm_bias_broadcast_over_rows(streamk):
    m, n, k = 200, 330, 512
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "N")
    bias = torch.randn(n, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda() * 4
    c = tb.addmm(bias, a, b, enable_streamk=streamk)
    assert_close_to_oracle(c, a, b, bias=bias, what="addmm")
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    assert tb.addmm(bias, a, b, out=out) is None
    assert torch.equal(out, tb.addmm(bias, a, b))


def test_errors_match_reference_behaviour():
    a = torch.randn(8, 16, device="cuda", dtype=torch.float16)
    b = torch.randn(32, 8, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError, match="Incompatible"):
        tb.matmul(a, b)
    a = torch.randn(8, 32, device="cuda", dtype=torch.float16, requires_grad=True)
    out = torch.empty(8, 8, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="don't support automatic differentiation"):
        tb.matmul(a, b, out=out)
    with pytest.raises(RuntimeError, match="don't support automatic differentiation"):
        tb.addmm(torch.zeros(8, device="cuda", dtype=torch.float16), a, b, out=out)


def test_backward_matches_torch_autograd_formulas():
    m, n, k = 128, 192, 256
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "N", seed=4)
    a.requires_grad_(True)
    b.requires_grad_(True)
    bias = torch.zeros(n, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    c = tb.addmm(bias, a, b)
    g = torch.randn(m, n, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).cuda()
    c.backward(g)
    assert_close_to_oracle(a.grad, g, b.detach().T, what="grad_a")
    assert_close_to_oracle(b.grad, a.detach().T, g, what="grad_b")
    assert torch.allclose(bias.grad.float().cpu(), g.float().sum(0).cpu(), rtol=1e-2, atol=1e-1)


def test_torch_compile_fullgraph():
    a, b = make_operands(256, 256, 256, torch.bfloat16, "T", "N")
    fn = torch.compile(lambda x, y: tb.matmul(x, y), fullgraph=True)
    assert_close_to_oracle(fn(a, b), a, b, what="compiled")


@pytest.mark.parametrize("streamk", [False, True])
@pytest.mark.parametrize("ta,tb_", LAYOUTS)
@pytest.mark.parametrize("m", [1, 5, 16, 33, 64])
def test_decode_shapes_take_the_transposed_path(m, ta, tb_, streamk):
    """Few rows of A against a wide B: the library computes C^T = B^T A^T internally; results, bias axis and output
    layout must be unaffected."""
    n, k = 1280, 512
    a, b = make_operands(m, n, k, torch.bfloat16, ta, tb_, seed=m)
    sel = tb.OrigamiMatmulSelector(m, n, k, torch.bfloat16, torch.bfloat16, torch.bfloat16, torch.device("cuda", 0),
                                   streamk=streamk)
    assert sel._cfg.swap_ab == 1
    c = tb.matmul(a, b, enable_streamk=streamk)
    assert_close_to_oracle(c, a, b, what=f"decode m={m} {ta}{tb_} sk={streamk}")
    bias = torch.randn(n, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    c2 = tb.addmm(bias, a, b, enable_streamk=streamk)
    assert_close_to_oracle(c2, a, b, bias=bias, what=f"decode addmm m={m}")


def test_decode_shape_a8w8_scales_swap_with_operands():
    from tritonblas_b200 import utils
    m, n, k = 16, 2048, 1024
    g = torch.Generator().manual_seed(0)
    a16 = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b16 = (torch.randn(k, n, generator=g) * 0.02).to(torch.bfloat16).cuda()
    a8, a_s = utils.quantize_tensor_per_channel(a16, torch.float8_e4m3fn, axis=1)
    b8, b_s = utils.quantize_tensor_per_channel(b16, torch.float8_e4m3fn, axis=0)
    b8 = b8.T.contiguous().T
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_a8w8(a8, b8, a_s, b_s, c)
    assert_close_to_oracle(c, a8, b8, a_scale=a_s, b_scale=b_s, what="decode a8w8")


def test_stream_order_is_kept_with_early_kernel_launch():
    """GEMM launches may be scheduled before the previous kernel of the stream has finished (programmatic dependent
    launch); they must still see everything enqueued before them: chained GEMMs, async host copies, torch kernels."""
    m = n = k = 512
    g = torch.Generator().manual_seed(77)
    b1 = (torch.randn(k, n, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b2 = (torch.randn(n, n, generator=g) * 0.05).to(torch.bfloat16).cuda()
    a_dev = torch.empty(m, k, dtype=torch.bfloat16, device="cuda")
    hosts = [(torch.randn(m, k, generator=g)).to(torch.bfloat16).pin_memory() for _ in range(12)]
    outs = []
    for h in hosts:
        a_dev.copy_(h, non_blocking=True)          # copy -> GEMM -> GEMM -> torch kernel -> GEMM, all on one stream
        c1 = tb.matmul(a_dev, b1)
        c2 = tb.matmul(c1, b2)
        c3 = tb.matmul(torch.relu(c2), b2)
        outs.append(c3)
    torch.cuda.synchronize()
    for h, c3 in zip(hosts, outs):
        r1 = (h.float() @ b1.float().cpu()).to(torch.bfloat16)
        r2 = (r1.float() @ b2.float().cpu()).to(torch.bfloat16)
        r3 = torch.relu(r2).float() @ b2.float().cpu()
        err = (c3.float().cpu() - r3).abs().max().item()
        assert err <= 3e-2 * r3.abs().max().item() + 1e-3, err
