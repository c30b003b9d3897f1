"""FP8 e4m3 a8w8 GEMM with per-token x per-channel fp32 scales fused in the epilogue, against the CPU oracle
(fp8 codes up-cast to fp32, product, * a_scale[:, None] * b_scale[None, :], cast; the intended semantics stated in the
reference's tests/test_matmul_a8w8_lt.py:11-38). Tolerance: rtol 1e-2 of the dequantised fp32 product plus 1e-2 of its
rms, for bf16/fp16/fp32 outputs (same codes on both sides, so only accumulation order and the output cast differ);
fp8 outputs: within one e4m3 step (rtol 0.125)."""
import pytest
import torch

import tritonblas_b200 as tb
from tests._util import assert_close_to_oracle
from tritonblas_b200 import utils

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


def _inputs(m, n, k, ta, tb_, seed=0):
    ga, gb = torch.Generator().manual_seed(seed), torch.Generator().manual_seed(seed + 10000)
    a16 = torch.randn(m, k, generator=ga).to(torch.bfloat16).cuda()
    b16 = (torch.randn(k, n, generator=gb) * 0.02).to(torch.bfloat16).cuda()
    a8, a_s = utils.quantize_tensor_per_channel(a16, FP8, axis=1)     # per token
    b8, b_s = utils.quantize_tensor_per_channel(b16, FP8, axis=0)     # per output channel
    if ta == "N":
        a8 = a8.T.contiguous().T
    b8 = b8.T.contiguous().T if tb_ == "T" else b8.contiguous()
    return a8, b8, a_s, b_s


@pytest.fixture(autouse=True)
def _no_device_failure():
    yield
    assert tb.device_status() == 0


@pytest.mark.parametrize("streamk", [False, True])
@pytest.mark.parametrize("ta,tb_", [("T", "T"), ("T", "N"), ("N", "T"), ("N", "N")])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (512, 384, 1024), (100, 200, 512)])
def test_a8w8_layouts(m, n, k, ta, tb_, streamk):
    a8, b8, a_s, b_s = _inputs(m, n, k, ta, tb_)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_a8w8(a8, b8, a_s, b_s, c, enable_streamk=streamk)
    assert_close_to_oracle(c, a8, b8, a_scale=a_s, b_scale=b_s, what=f"a8w8 {(m, n, k)} {ta}{tb_} sk={streamk}")


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32, FP8])
def test_a8w8_output_types(out_dtype):
    m, n, k = 256, 512, 512
    a8, b8, a_s, b_s = _inputs(m, n, k, "T", "T", seed=3)
    c = torch.empty(m, n, dtype=out_dtype, device="cuda")
    sel = tb.OrigamiMatmulSelector(m, n, k, FP8, FP8, out_dtype, torch.device("cuda", 0))
    tb.matmul_a8w8_lt(a8, b8, a_s, b_s, c, sel, tb.matmul_preamble(sel))
    assert_close_to_oracle(c, a8, b8, a_scale=a_s, b_scale=b_s, rtol=0.125 if out_dtype == FP8 else 1e-2,
                           what=f"a8w8 out={out_dtype}")


@pytest.mark.parametrize("m", [16, 256, 4096])
def test_a8w8_config3_shapes(m):
    """BASELINE config 3: M in {16, 256, 4096}, N = 28672, K = 8192, bf16 out; 384 sampled output columns checked."""
    n, k = 28672, 8192
    a8, b8, a_s, b_s = _inputs(m, n, k, "T", "T", seed=m)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_a8w8(a8, b8, a_s, b_s, c, enable_streamk=(m <= 256))
    cols = torch.randint(0, n, (380,), generator=torch.Generator().manual_seed(9))
    cols = torch.cat([cols, torch.tensor([0, 255, 256, n - 1])]).cuda()
    rows = None if m <= 256 else torch.randint(0, m, (64,), generator=torch.Generator().manual_seed(10)).tolist()
    assert_close_to_oracle(c[:, cols], a8, b8[:, cols], a_scale=a_s, b_scale=b_s[cols], rows=rows, what=f"cfg3 m={m}")


@pytest.mark.parametrize("streamk", [False, True])
@pytest.mark.parametrize("ta,tb_", [("T", "T"), ("N", "N")])
@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (100, 200, 1024), (16, 1024, 2048)])
def test_int8_a8w8(m, n, k, ta, tb_, streamk):
    """INT8 operands, int32 accumulation on the tensor cores, per-row x per-column fp32 scales, bf16 output."""
    g = torch.Generator().manual_seed(m + k)
    a16 = torch.randn(m, k, generator=g).cuda()
    b16 = (torch.randn(k, n, generator=g) * 0.02).cuda()
    a8, a_s = utils.quantize_tensor_per_channel(a16, torch.int8, axis=1)
    b8, b_s = utils.quantize_tensor_per_channel(b16, torch.int8, axis=0)
    if ta == "N":
        a8 = a8.T.contiguous().T
    b8 = b8.T.contiguous().T if tb_ == "T" else b8.contiguous()
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_a8w8(a8, b8, a_s, b_s, c, enable_streamk=streamk)
    assert_close_to_oracle(c, a8, b8, a_scale=a_s, b_scale=b_s, what=f"int8 {(m, n, k)} {ta}{tb_} sk={streamk}")


def test_int8_output_saturates():
    m, n, k = 128, 256, 256
    g = torch.Generator().manual_seed(2)
    a8 = torch.randint(-127, 128, (m, k), generator=g, dtype=torch.int8).cuda()
    b8 = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda().T
    a_s = torch.full((m,), 1e-3, device="cuda")
    b_s = torch.full((n,), 1.0, device="cuda")
    c = torch.empty(m, n, dtype=torch.int8, device="cuda")
    tb.matmul_a8w8(a8, b8, a_s, b_s, c)
    from oracle import gemm_oracle
    ref = gemm_oracle.gemm_ref(a8, b8, torch.int8, a_s, b_s)
    diff = (c.cpu().int() - ref.int()).abs()
    assert diff.max() <= 1 and (diff > 0).float().mean() < 0.01     # ties may round differently at .5 exactly
    assert c.max() == 127 or c.min() == -128 or ref.abs().max() < 127


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,k", [(1, 8), (37, 264), (256, 8192), (1000, 1536)])
def test_fp8_row_quantiser_is_bit_exact_against_the_oracle(rows, k, dtype):
    """The CUDA quantiser against the CPU oracle's restatement of the reference fixture (utils.py:340-377), and the
    package's torch fixture against the same oracle, so all three agree bit for bit."""
    g = torch.Generator().manual_seed(rows + k)
    x = (torch.randn(rows, k, generator=g) * 3).to(dtype).cuda()
    x[0, 0] = 0.0
    if rows > 2:
        x[2] = 0.0                                    # all-zero row: scale clamps at 1e-8 / 448
    q, s = utils.quantize_fp8_rows(x)
    from oracle import gemm_oracle
    q_ref, s_ref = gemm_oracle.quantize_per_channel_ref(x, FP8, axis=1)
    assert torch.equal(s.cpu(), s_ref)
    assert torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))
    q_fix, s_fix = utils.quantize_tensor_per_channel(x, FP8, axis=1)
    assert torch.equal(s_fix.cpu().reshape(-1), s_ref)
    assert torch.equal(q_fix.cpu().view(torch.uint8), q_ref.view(torch.uint8))
