"""MXFP4 quantiser and fused Hadamard+quantiser kernels: codes and scales must be bit-exact against the CPU oracle
(which is itself pinned bit-for-bit to the reference quantiser by tests/test_oracle_golden.py)."""
import os

import numpy as np
import pytest
import torch

import tritonblas_b200 as tb
from oracle import mxfp4_oracle
from tritonblas_b200 import utils

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _check(x_cpu, dtype, hadamard):
    x = x_cpu.to(dtype).cuda()
    fn = utils.hadamard_mxfp4_quant if hadamard else utils.dynamic_mxfp4_quant
    codes, scales = fn(x)
    xf = x.float().cpu().numpy()
    ref = mxfp4_oracle.hadamard_quantize_mxfp4(xf) if hadamard else mxfp4_oracle.quantize_mxfp4(xf)
    assert np.array_equal(scales.cpu().numpy(), ref[1]), "scale bytes differ"
    assert np.array_equal(codes.cpu().numpy(), ref[0]), "code bytes differ"


def test_golden_inputs_match_reference_kernel_outputs():
    """Straight against what the reference's own kernel produced (fp32 inputs)."""
    g = np.load(os.path.join(GOLDEN, "mxfp4_quant.npz"))
    for name in sorted(k[:-2] for k in g.files if k.endswith("_x")):
        codes, scales = utils.dynamic_mxfp4_quant(torch.from_numpy(g[name + "_x"]).cuda())
        assert np.array_equal(scales.cpu().numpy(), g[name + "_scales"]), name
        assert np.array_equal(codes.cpu().numpy(), g[name + "_codes"]), name


@pytest.mark.parametrize("hadamard", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(1, 32), (7, 96), (128, 256), (333, 1024), (1000, 4096)])
def test_bit_exact_random(shape, dtype, hadamard):
    g = torch.Generator().manual_seed(shape[0] * 7 + shape[1])
    _check(torch.randn(*shape, generator=g), dtype, hadamard)


@pytest.mark.parametrize("hadamard", [False, True])
def test_bit_exact_edge_values(hadamard):
    g = torch.Generator().manual_seed(5)
    x = torch.randn(16, 128, generator=g)
    x[0] = 0.0                       # all-zero blocks -> scale byte 0, codes 0
    x[1, :32] = 0.0
    x[2] *= 1e-30
    x[3] *= 1e30
    x[4, :8] = torch.tensor([0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    x[5, :32] = 6.0
    x[6, :32] = -6.0
    x[7, :32] = torch.linspace(-7.0, 7.0, 32)
    x[8, :32] = 7.0
    x[9, :32] = 6.9999995
    x[10] *= 1e-38                   # fp32 denormals
    x[11, 3] = 3.0e38
    _check(x, torch.float32, hadamard)
    _check(x.clamp(-6e4, 6e4), torch.float16, hadamard)
    _check(x, torch.bfloat16, hadamard)


def test_strided_rows_and_empty():
    g = torch.Generator().manual_seed(1)
    big = torch.randn(64, 512, generator=g).to(torch.bfloat16).cuda()
    view = big[:, 128:384]           # row stride 512 elements, 16-byte aligned start
    codes, scales = utils.dynamic_mxfp4_quant(view)
    ref = mxfp4_oracle.quantize_mxfp4(view.float().cpu().numpy())
    assert np.array_equal(codes.cpu().numpy(), ref[0]) and np.array_equal(scales.cpu().numpy(), ref[1])
    c, s = utils.dynamic_mxfp4_quant(torch.empty(0, 64, dtype=torch.bfloat16, device="cuda"))
    assert c.shape == (0, 32) and s.shape == (0, 2)


def test_full_size_activation_8192_square():
    """BASELINE config 4 activation: bf16 N(0,1) 8192 x 8192. The oracle checks 64 sampled rows bit-exactly; the rest is
    covered by size-independent properties: every scale is the exponent rule applied to its own block (recomputed with
    torch on the GPU from the rotated values' block maxima), and dequantised values are within half a code step."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(8192, 8192, generator=g).to(torch.bfloat16).cuda()
    codes, scales = utils.hadamard_mxfp4_quant(x)
    rows = torch.randint(0, 8192, (64,), generator=g)
    ref = mxfp4_oracle.hadamard_quantize_mxfp4(x[rows.cuda()].float().cpu().numpy())
    assert np.array_equal(codes[rows.cuda()].cpu().numpy(), ref[0])
    assert np.array_equal(scales[rows.cuda()].cpu().numpy(), ref[1])
    # properties over the whole matrix
    deq = utils.mxfp4_to_f32(codes) * utils.e8m0_to_f32(scales).repeat_interleave(32, dim=1)
    assert torch.isfinite(deq).all()
    # the rotation is orthonormal: block energies are preserved up to quantisation error
    e_in = x.float().pow(2).sum().item()
    e_out = deq.pow(2).sum().item()
    assert abs(e_out - e_in) / e_in < 0.02
    # quantisation error per element is at most half the largest code step (1.0 between 4 and 6, 2.0 at the clamp) x scale
    plain_codes, plain_scales = utils.dynamic_mxfp4_quant(x)
    deq_plain = utils.mxfp4_to_f32(plain_codes) * utils.e8m0_to_f32(plain_scales).repeat_interleave(32, dim=1)
    step = utils.e8m0_to_f32(plain_scales).repeat_interleave(32, dim=1)
    assert ((deq_plain - x.float()).abs() <= 1.0 * step + 1e-6).all()
    assert tb.device_status() == 0
