"""MXFP4 GEMM (block-scaled tensor-core instruction) against the dequantised fp32 product of the CPU oracle
(the check the reference's tests/test_matmul_fp4.py:20-46 builds, here asserted numerically).
Tolerance: both sides multiply the same e2m1 codes and e8m0 scales exactly and accumulate in fp32, so only
accumulation order and the bf16 output cast differ: rtol 1e-2 plus 1e-2 of the reference's rms."""
import numpy as np
import pytest
import torch

import tritonblas_b200 as tb
from oracle import mxfp4_oracle
from tritonblas_b200 import utils

pytestmark = pytest.mark.gpu


def _quantised(m, n, k, seed=0, hadamard=False):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=g).to(torch.bfloat16).cuda()
    q = utils.hadamard_mxfp4_quant if hadamard else utils.dynamic_mxfp4_quant
    return a, b, q(a), q(b)


def _check(c, qa, sa, qb, sb, what, rows=None, cols=None):
    qa, sa, qb, sb = (t.cpu().numpy() for t in (qa, sa, qb, sb))
    got = c.float().cpu().numpy()
    if rows is not None:
        qa, sa, got = qa[rows], sa[rows], got[rows]
    if cols is not None:
        qb, sb, got = qb[cols], sb[cols], got[:, cols]
    ref = mxfp4_oracle.mxfp4_gemm_ref(qa, sa, qb, sb)
    rms = float(np.sqrt((ref ** 2).mean()))
    err = np.abs(got - ref)
    bad = err > 1e-2 * np.abs(ref) + 1e-2 * rms
    assert np.isfinite(got).all(), what
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} off, max err {err.max():.4g}, rms {rms:.4g}, first {np.argwhere(bad)[0]}"


@pytest.fixture(autouse=True)
def _no_device_failure():
    yield
    assert tb.device_status() == 0


@pytest.mark.parametrize("block_m,block_n", [(128, 64), (128, 128), (128, 192), (256, 64), (256, 128), (256, 192), (None, None)])
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (256, 256, 512), (512, 448, 1024), (384, 640, 2048)])
def test_fp4_tile_shapes(m, n, k, block_m, block_n):
    _, _, (qa, sa), (qb, sb) = _quantised(m, n, k, seed=m + n)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb, block_m=block_m, block_n=block_n, block_k=256 if block_m else None)
    _check(c, qa, sa, qb, sb, f"fp4 {(m, n, k)} tile {block_m}x{block_n}")


@pytest.mark.parametrize("m,n,k", [(100, 72, 256), (130, 260, 96), (1, 33, 64), (257, 129, 32), (333, 500, 1120)])
def test_fp4_ragged_shapes_and_k_tails(m, n, k):
    _, _, (qa, sa), (qb, sb) = _quantised(m, n, k, seed=k)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb)
    _check(c, qa, sa, qb, sb, f"fp4 ragged {(m, n, k)}")


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_fp4_output_types(out_dtype):
    m, n, k = 256, 384, 512
    _, _, (qa, sa), (qb, sb) = _quantised(m, n, k, seed=4)
    c = torch.empty(m, n, dtype=out_dtype, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb)
    _check(c, qa, sa, qb, sb, f"fp4 out {out_dtype}")


def test_fp4_extreme_scales():
    """Scale bytes across the e8m0 range (kept finite): tiny and huge block scales must combine exactly."""
    m, n, k = 128, 128, 256
    _, _, (qa, sa), (qb, sb) = _quantised(m, n, k, seed=8)
    g = torch.Generator().manual_seed(3)
    sa = torch.randint(100, 150, sa.shape, generator=g, dtype=torch.uint8).cuda()
    sb = torch.randint(100, 150, sb.shape, generator=g, dtype=torch.uint8).cuda()
    c = torch.empty(m, n, dtype=torch.float32, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb)
    _check(c, qa, sa, qb, sb, "fp4 wide scales")


def test_fp4_config4_full_size_with_hadamard_activations():
    """BASELINE config 4: 8192^3, bf16 N(0,1) sources; A through the fused Hadamard+quantise kernel, B through the same
    rotation offline. 32 sampled rows x 256 sampled columns against the oracle, and the rotation identity
    (A H)(B H)^T ~= A B^T checked against the bf16 source product within the quantisation error."""
    m = n = k = 8192
    a, b, (qa, sa), (qb, sb) = _quantised(m, n, k, seed=11, hadamard=True)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb)
    g = torch.Generator().manual_seed(12)
    rows = torch.randint(0, m, (32,), generator=g).numpy()
    cols = torch.randint(0, n, (256,), generator=g).numpy()
    _check(c, qa, sa, qb, sb, "fp4 8192^3", rows=rows, cols=cols)
    src = a[torch.as_tensor(rows).cuda()].float() @ b[torch.as_tensor(cols).cuda()].float().T
    got = c[torch.as_tensor(rows).cuda()][:, torch.as_tensor(cols).cuda()].float()
    rel = (got - src).norm() / src.norm()
    assert rel < 0.2, rel   # 4-bit operands: ~10 % relative Frobenius error is expected, 100 % would mean a layout bug


@pytest.mark.parametrize("rows,k", [(1, 32), (130, 96), (256, 1024), (333, 1120)])
def test_scale_atoms_round_trip_and_fused_emit(rows, k):
    """Atom-ordered scales: the re-arrangement kernel, the quantiser's direct emit and the row-major bytes all agree."""
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16).cuda()
    codes, scales = utils.dynamic_mxfp4_quant(x)
    codes2, atoms = utils.dynamic_mxfp4_quant(x, scale_atoms=True)
    assert torch.equal(codes, codes2)
    assert torch.equal(atoms.to_row_major(), scales)
    conv = utils.mxfp4_scales_to_atoms(scales, k)
    assert torch.equal(conv.to_row_major(), scales)
    assert torch.equal(conv.data, atoms.data)            # padding bytes included (127)


def test_fp4_accepts_prearranged_scales():
    m, n, k = 384, 448, 1024
    g = torch.Generator().manual_seed(21)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=g).to(torch.bfloat16).cuda()
    qa, sa = utils.hadamard_mxfp4_quant(a, scale_atoms=True)
    qb, sb = utils.hadamard_mxfp4_quant(b, scale_atoms=True)
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tb.matmul_fp4(qa, qb, c, sa, sb)
    _check(c, qa, sa.to_row_major(), qb, sb.to_row_major(), "fp4 atoms in")
