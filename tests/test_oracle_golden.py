"""The CPU oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""
import os

import numpy as np
import torch

from oracle import gemm_oracle, mxfp4_oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_e2m1_decoder_matches_reference_table():
    g = np.load(os.path.join(GOLDEN, "decoders.npz"))
    got = mxfp4_oracle.decode_e2m1(g["bytes"])
    assert np.array_equal(got.view(np.uint32), g["e2m1"].view(np.uint32))  # bit-exact, including -0.0


def test_e8m0_decoder_matches_reference_bits():
    g = np.load(os.path.join(GOLDEN, "decoders.npz"))
    got = mxfp4_oracle.decode_e8m0(g["bytes"])
    assert np.array_equal(got.view(np.uint32), g["e8m0_bits"])
    assert got[0, 127] == 1.0 and got[0, 0] == np.float32(2.0 ** -127) and np.isnan(got[0, 255])


def test_quantiser_bit_exact_against_reference_kernel():
    g = np.load(os.path.join(GOLDEN, "mxfp4_quant.npz"))
    names = sorted(k[:-2] for k in g.files if k.endswith("_x"))
    assert len(names) >= 6
    for name in names:
        codes, scales = mxfp4_oracle.quantize_mxfp4(g[name + "_x"])
        assert np.array_equal(scales, g[name + "_scales"]), name
        assert np.array_equal(codes, g[name + "_codes"]), name


def test_quantiser_known_answer():
    # block maximum 5.0 -> scale byte 127 (2^0); ties round away from zero: 0.25->0.5, 0.75->1, 1.25->1.5, 1.75->2 ...
    x = np.zeros((1, 32), np.float32)
    x[0, :8] = [0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    codes, scales = mxfp4_oracle.quantize_mxfp4(x)
    assert scales.tolist() == [[127]]
    assert mxfp4_oracle.dequantize_mxfp4(codes, scales)[0, :8].tolist() == [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_quantiser_zero_block_and_ragged_rows():
    x = np.zeros((3, 64), np.float32)
    x[1, 40] = -1.0
    codes, scales = mxfp4_oracle.quantize_mxfp4(x)
    assert scales[0].tolist() == [0, 0] and not codes[0].any()
    assert codes.shape == (3, 32) and scales.shape == (3, 2)
    deq = mxfp4_oracle.dequantize_mxfp4(codes, scales)
    assert deq[1, 40] == -1.0


def test_hadamard_is_orthonormal_sylvester():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8, 96)).astype(np.float32)
    y = mxfp4_oracle.hadamard32(x)
    # involution up to fp32 rounding, and the first output of each block is the scaled block sum
    assert np.allclose(mxfp4_oracle.hadamard32(y), x, atol=1e-5)
    assert np.allclose(y[:, 0], x[:, :32].sum(1) / np.sqrt(32), atol=1e-5)
    # natural (Sylvester) ordering: output 1 is sum of even minus sum of odd inputs
    assert np.allclose(y[:, 1], (x[:, 0:32:2].sum(1) - x[:, 1:32:2].sum(1)) / np.sqrt(32), atol=1e-5)


def test_gemm_oracle_against_reference_monolithic_kernel():
    g = np.load(os.path.join(GOLDEN, "gemm_monolithic.npz"))
    for tag in ("f16", "f16_ragged"):
        a = torch.from_numpy(g[tag + "_a"]).view(torch.float16)
        b = torch.from_numpy(g[tag + "_b"]).view(torch.float16)
        c = torch.from_numpy(g[tag + "_c"]).view(torch.float16)
        ref = gemm_oracle.gemm_ref(a, b, torch.float16)
        # both sides accumulate in fp32 and round once to fp16: allow one fp16 ulp at the largest magnitude
        assert torch.allclose(ref.float(), c.float(), rtol=2e-3, atol=2e-3), tag


def test_gemm_oracle_epilogue_order():
    a = torch.tensor([[1.0, 2.0]], dtype=torch.float16)
    b = torch.tensor([[3.0], [4.0]], dtype=torch.float16)
    out = gemm_oracle.gemm_ref(a, b, torch.float32, a_scale=torch.tensor([0.5]), b_scale=torch.tensor([4.0]),
                               bias=torch.tensor([1.0]))
    assert out.item() == (11.0 * 0.5) * 4.0 + 1.0


def test_mxfp4_gemm_oracle_small():
    rng = np.random.default_rng(1)
    a = rng.standard_normal((4, 64)).astype(np.float32)
    b = rng.standard_normal((5, 64)).astype(np.float32)
    qa, sa = mxfp4_oracle.quantize_mxfp4(a)
    qb, sb = mxfp4_oracle.quantize_mxfp4(b)
    got = mxfp4_oracle.mxfp4_gemm_ref(qa, sa, qb, sb)
    want = mxfp4_oracle.dequantize_mxfp4(qa, sa) @ mxfp4_oracle.dequantize_mxfp4(qb, sb).T
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)
