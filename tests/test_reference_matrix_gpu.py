"""The reference's own test matrix, run through the reference's package name (``import tritonblas``) and checked against
the CPU oracle instead of torch on the GPU.

  * examples/example_matmul.py:8-17 and examples/example_matmul_lt.py:8-19: the documented call sequences;
  * tests/test_matmul.py:9-51 and tests/test_matmul_lt.py:9-58: full-size shapes, incl. K = 970132 (not a multiple of 8,
    15 159 K blocks) x {fp16, bf16, fp32} x four operand layouts x {persistent, stream-K, work-stealing};
  * tests/test_matmul_correctness.py:24-130 and tests/test_addmm_correctness.py: forward and backward, eager and
    torch.compile(fullgraph=True), with stream-K and work-stealing switched on and off.

Full-size products are checked on sampled rows x sampled columns (the oracle is a CPU fp32 product). Tolerance: rtol 1e-2
plus 1e-2 of the reference's rms for 16-bit outputs and tf32 products, 1e-4 for exact fp32 products.
"""
import pytest
import torch

import tritonblas
from tritonblas.utils import generate_matmul_inputs
from oracle import gemm_oracle

pytestmark = pytest.mark.gpu

LAYOUTS = [("T", "T"), ("N", "N"), ("T", "N"), ("N", "T")]
MODES = ["persistent", "streamk", "work_stealing"]
DTYPES = [torch.float16, torch.bfloat16, torch.float32]
# reference conftest.py:40-66
STANDARD_DIMS = [(128, 256, 512), (256, 256, 256), (512, 1024, 768), (768, 1024, 512), (2048, 1024, 512), (1024, 2048, 512)]
EDGE_CASE_DIMS = [(32, 32, 32), (64, 16, 128), (16, 64, 128), (128, 8, 256), (8, 128, 256), (12, 12, 512), (15, 17, 512),
                  (19, 13, 512), (128, 64, 12)]
SKINNY_DIMS = [(16, 16, 4096), (32, 32, 8192)]


@pytest.fixture(autouse=True)
def _no_device_failure():
    yield
    assert tritonblas.device_status() == 0


def _check_sampled(c, a, b, rtol, what, nrows=24, ncols=96, bias=None):
    """Compare C[rows][:, cols] with the oracle's A[rows] @ B[:, cols] (fp32 accumulate on the CPU)."""
    m, n = c.shape
    g = torch.Generator().manual_seed(m * 31 + n)
    rows = torch.unique(torch.cat([torch.randint(0, m, (nrows,), generator=g), torch.tensor([0, m - 1, min(m - 1, 127), min(m - 1, 128)])]))
    cols = torch.unique(torch.cat([torch.randint(0, n, (ncols,), generator=g), torch.tensor([0, n - 1, min(n - 1, 255), min(n - 1, 256)])]))
    rows_d, cols_d = rows.to(c.device), cols.to(c.device)
    a_s = a[rows_d].contiguous()
    b_s = b[:, cols_d].contiguous()
    ref = gemm_oracle.gemm_ref_f32(a_s, b_s, bias=bias[cols_d] if bias is not None else None)
    got = c[rows_d][:, cols_d].float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs()
    bad = err > rtol * ref.abs() + rtol * max(rms, 1e-30)
    assert torch.isfinite(got).all(), what
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} sampled elements off, max err {err.max().item():.4g}, rms {rms:.4g}"


def test_example_matmul_call_sequence():
    """examples/example_matmul.py:8-17 (smaller m, n, k): positional out argument, result in C."""
    m, n, k = 1024, 768, 512
    A = torch.randn(m, k, device="cuda", dtype=torch.float16)
    B = torch.randn(n, k, device="cuda", dtype=torch.float16).T
    C = torch.zeros((m, n), device="cuda", dtype=torch.float16)
    assert tritonblas.matmul(A, B, C) is None
    _check_sampled(C, A, B, 1e-2, "example_matmul")


def test_example_matmul_lt_call_sequence():
    """examples/example_matmul_lt.py:8-19: selector, preamble, matmul_lt."""
    m, n, k = 1024, 768, 512
    A = torch.randn(m, k, device="cuda", dtype=torch.float16)
    B = torch.randn(n, k, device="cuda", dtype=torch.float16).T
    C = torch.zeros((m, n), device="cuda", dtype=torch.float16)
    selector = tritonblas.OrigamiMatmulSelector(m, n, k, A.dtype, B.dtype, C.dtype, A.device)
    config = tritonblas.matmul_preamble(selector)
    tritonblas.matmul_lt(A, B, C, selector, config)
    _check_sampled(C, A, B, 1e-2, "example_matmul_lt")


def test_do_bench_times_a_launch():
    A = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16)
    B = torch.randn(512, 512, device="cuda", dtype=torch.bfloat16).T
    C = torch.empty(512, 512, device="cuda", dtype=torch.bfloat16)
    selector = tritonblas.OrigamiMatmulSelector(512, 512, 512, A.dtype, B.dtype, C.dtype, A.device)
    config = tritonblas.matmul_preamble(selector)
    ms = tritonblas.do_bench(lambda: tritonblas.matmul_lt(A, B, C, selector, config), reset_fn=lambda: config.reset(),
                             n_warmup=2, n_repeat=5)
    assert 0 < ms < 50
    lo, hi = tritonblas.do_bench(lambda: tritonblas.matmul_lt(A, B, C, selector, config), n_warmup=1, n_repeat=5,
                                 quantiles=[0.0, 1.0])
    assert 0 < lo <= hi


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("transA,transB", LAYOUTS)
@pytest.mark.parametrize("dtype", DTYPES, ids=["fp16", "bf16", "fp32"])
@pytest.mark.parametrize("m,n,k", [(8192, 8192, 8192), (4864, 8192, 4160), (4096, 4096, 4096), (512, 2048, 970132)])
def test_matmul_lt_full_size_matrix(m, n, k, dtype, transA, transB, mode):
    """tests/test_matmul_lt.py:9-58 of the reference at its own sizes (tests/test_matmul.py:9-51 runs the first three
    through tritonblas.matmul; the sequence below is the _lt one and the last assertion covers the plain entry point)."""
    enable_streamk = mode == "streamk"
    work_stealing = mode == "work_stealing"
    # randn products at K = 970132 have a standard deviation near 1000, inside fp16's range
    inputs = generate_matmul_inputs(m, n, k, dtype, dtype, transA, transB, "randn", seed=7)
    selector = tritonblas.OrigamiMatmulSelector(m, n, k, inputs.A.dtype, inputs.B.dtype, inputs.C.dtype, inputs.A.device,
                                                streamk=enable_streamk)
    config = tritonblas.matmul_preamble(selector)
    tritonblas.matmul_lt(inputs.A, inputs.B, inputs.C, selector, config, enable_streamk, work_stealing=work_stealing)
    rtol = 1e-4 if dtype == torch.float32 else 1e-2     # fp32 operands: exact fp32 products unless torch allows tf32
    _check_sampled(inputs.C, inputs.A, inputs.B, rtol, f"{(m, n, k)} {dtype} {transA}{transB} {mode}")
    if (m, n, k) == (4096, 4096, 4096) and dtype != torch.float32:
        out = torch.empty_like(inputs.C)
        tritonblas.matmul(inputs.A, inputs.B, out, enable_streamk=enable_streamk, work_stealing=work_stealing)
        assert torch.equal(out, inputs.C)            # same kernel, same schedule: identical bits


def _fn(name, use_compile):
    f = getattr(tritonblas, name)
    return torch.compile(f, fullgraph=True) if use_compile else f


@pytest.mark.parametrize("work_stealing", [False, True])
@pytest.mark.parametrize("enable_streamk", [False, True])
@pytest.mark.parametrize("m,n,k", STANDARD_DIMS + EDGE_CASE_DIMS + SKINNY_DIMS)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_matmul_and_addmm_forward_backward_eager(m, n, k, dtype, enable_streamk, work_stealing):
    """tests/test_matmul_correctness.py:24-130 and tests/test_addmm_correctness.py, eager: forward and both gradients
    (and the bias gradient) against the oracle."""
    g = torch.Generator(device="cuda").manual_seed(42)
    a = torch.randn(m, k, device="cuda", dtype=dtype, generator=g, requires_grad=True)
    b = torch.randn(k, n, device="cuda", dtype=dtype, generator=g, requires_grad=True)
    bias = torch.randn(n, device="cuda", dtype=dtype, generator=g, requires_grad=True)
    go = torch.randn(m, n, device="cuda", dtype=dtype, generator=g)
    for name in ("matmul", "addmm"):
        a.grad = b.grad = bias.grad = None
        if name == "matmul":
            out = tritonblas.matmul(a, b, enable_streamk=enable_streamk, work_stealing=work_stealing)
            ref = gemm_oracle.gemm_ref_f32(a, b)
        else:
            out = tritonblas.addmm(bias, a, b, enable_streamk=enable_streamk, work_stealing=work_stealing)
            ref = gemm_oracle.gemm_ref_f32(a, b, bias=bias)
        _close(out, ref, f"{name} forward")
        out.backward(go)
        _close(a.grad, gemm_oracle.gemm_ref_f32(go, b.detach().T), f"{name} grad_a")
        _close(b.grad, gemm_oracle.gemm_ref_f32(a.detach().T, go), f"{name} grad_b")
        if name == "addmm":
            _close(bias.grad, go.float().cpu().sum(0), "grad_bias", rtol=2e-2)


def _close(got, ref, what, rtol=1e-2):
    got = got.detach().float().cpu()
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs()
    assert bool((err <= rtol * ref.abs() + rtol * max(rms, 1e-30)).all()), f"{what}: max err {err.max().item():.4g}, rms {rms:.4g}"


@pytest.mark.parametrize("work_stealing", [False, True])
@pytest.mark.parametrize("enable_streamk", [False, True])
@pytest.mark.parametrize("name", ["matmul", "addmm"])
def test_compiled_forward_backward(name, enable_streamk, work_stealing):
    """torch.compile(fullgraph=True) x stream-K x work-stealing x backward (tests/test_matmul_correctness.py:24-28,60-96;
    the same for addmm), on a standard, an edge and a skinny shape."""
    import torch._dynamo
    torch._dynamo.config.cache_size_limit = 64
    fn = _fn(name, True)
    for (m, n, k) in [(512, 1024, 768), (15, 17, 512), (16, 16, 4096)]:
        g = torch.Generator(device="cuda").manual_seed(43)
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16, generator=g, requires_grad=True)
        b = torch.randn(k, n, device="cuda", dtype=torch.bfloat16, generator=g, requires_grad=True)
        bias = torch.randn(n, device="cuda", dtype=torch.bfloat16, generator=g, requires_grad=True)
        go = torch.randn(m, n, device="cuda", dtype=torch.bfloat16, generator=g)
        if name == "matmul":
            out = fn(a, b, enable_streamk=enable_streamk, work_stealing=work_stealing)
            ref = gemm_oracle.gemm_ref_f32(a, b)
        else:
            out = fn(bias, a, b, enable_streamk=enable_streamk, work_stealing=work_stealing)
            ref = gemm_oracle.gemm_ref_f32(a, b, bias=bias)
        _close(out, ref, f"compiled {name} forward {(m, n, k)}")
        out.backward(go)
        _close(a.grad, gemm_oracle.gemm_ref_f32(go, b.detach().T), f"compiled {name} grad_a {(m, n, k)}")
        _close(b.grad, gemm_oracle.gemm_ref_f32(a.detach().T, go), f"compiled {name} grad_b {(m, n, k)}")


@pytest.mark.parametrize("use_compile", [False, True])
@pytest.mark.parametrize("name", ["matmul", "addmm"])
def test_out_argument_with_grad_raises(name, use_compile):
    """tests/test_matmul_correctness.py:122-140: the error text is pinned by the reference's regex."""
    a = torch.randn(64, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(64, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    bias = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(64, 64, device="cuda", dtype=torch.bfloat16)
    fn = _fn(name, use_compile)
    with pytest.raises(RuntimeError, match="don't support automatic differentiation"):
        if name == "matmul":
            fn(a, b, out=out)
        else:
            fn(bias, a, b, out=out)
