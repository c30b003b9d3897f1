"""MXFP4 oracle: e2m1 / e8m0 decoders, the block-32 quantiser, the 32-point Hadamard rotation and the dequantised
fp32 GEMM (test infrastructure; see oracle/__init__.py). numpy integer arithmetic throughout, so results are exact.

Reference lines followed:
  decode_e2m1      include/tritonblas/utils.py:547-607   (nibble table, low nibble = even element)
  decode_e8m0      include/tritonblas/utils.py:610-643   (0 -> 2^-126 kept as bits 0x00400000, 255 -> NaN)
  quantize_mxfp4   include/tritonblas/utils.py:679-726   (amax -> pow2 round-up -> e8m0 -> e2m1 by bit operations)
  mxfp4_gemm_ref   tests/test_matmul_fp4.py:20-46        (dequantise, fp32 product)
"""
import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                       dtype=np.float32)
HADAMARD_SCALE = np.float32(0.17677669529663687)  # 1/sqrt(32)


def decode_e2m1(packed):
    """(rows, K/2) uint8 -> (rows, K) float32; element 2i is the low nibble of byte i."""
    packed = np.asarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.float32)
    out[..., 0::2] = E2M1_VALUES[packed & 0xF]
    out[..., 1::2] = E2M1_VALUES[packed >> 4]
    return out


def decode_e8m0(scales):
    """uint8 exponent bytes -> float32 2^(s-127); byte 0 decodes to the bit pattern 0x00400000, byte 255 to NaN."""
    s = np.asarray(scales, dtype=np.uint8)
    bits = s.astype(np.uint32) << 23
    bits = np.where(s == 0, np.uint32(0x00400000), bits)
    bits = np.where(s == 0xFF, np.uint32(0x7F800001), bits)
    return bits.astype(np.uint32).view(np.float32)


def dequantize_mxfp4(packed, scales):
    vals = decode_e2m1(packed)
    sc = np.repeat(decode_e8m0(scales), 32, axis=-1)
    return vals * sc


def quantize_mxfp4(x):
    """Quantise float32 x (rows, K), K % 32 == 0, to packed e2m1 codes (rows, K/2) and e8m0 scales (rows, K/32)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % 32 == 0
    xb = x.reshape(rows, K // 32, 32)
    amax = np.abs(xb).max(axis=-1, keepdims=True).astype(np.float32)
    # round the block maximum up to a power of two when its mantissa is >= 1.75
    abits = amax.view(np.int32).astype(np.int64)
    abits = (abits + 0x200000) & 0xFF800000
    amax_p2 = (abits & 0xFFFFFFFF).astype(np.uint32).view(np.float32)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(amax_p2)) - 2.0
    e = np.clip(e, -127.0, 127.0).astype(np.float32)
    # 2^-e applied as an exact fp32 multiply (for e = -127 the factor is 2^127)
    qx = (xb * np.exp2(-e).astype(np.float32)).astype(np.float32)
    scale_byte = ((e.astype(np.int32) + 127) & 0xFF).astype(np.uint8).reshape(rows, K // 32)

    bits = qx.view(np.uint32).astype(np.int64)
    sign = bits & 0x80000000
    ex = (bits >> 23) & 0xFF
    man = bits & 0x7FFFFF
    # values below 1.0: shift the mantissa (with its hidden one) down into the single e2m1 denormal bit position
    shift = np.clip(127 - (ex + 1), 0, 63)
    man = np.where(ex < 127, (0x400000 | (man >> 1)) >> shift, man)
    ex = np.maximum(ex, 126) - 126
    code = np.minimum((((ex << 2) | (man >> 21)) + 1) >> 1, 7)  # round to nearest, ties away from zero, saturate at 6.0
    code = ((sign >> 28) | code).astype(np.uint8).reshape(rows, K)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8)
    return packed, scale_byte


def hadamard32(x):
    """Rotate every 32 contiguous elements of each row by the Sylvester Hadamard matrix H32 / sqrt(32).

    Operation order is part of the contract (it decides the fp32 roundings): five in-place butterfly stages with
    strides 1, 2, 4, 8, 16, each (a, b) -> (a + b, a - b) in fp32 without fused multiply-add, then one fp32 multiply by
    0.17677669529663687. No reference implementation exists (parity unpinned); the CUDA kernel performs the same
    sequence.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % 32 == 0
    y = x.reshape(rows, K // 32, 32).copy()
    for stride in (1, 2, 4, 8, 16):
        v = y.reshape(rows, K // 32, 32 // (2 * stride), 2, stride)
        a = v[..., 0, :].copy()
        b = v[..., 1, :].copy()
        v[..., 0, :] = a + b
        v[..., 1, :] = a - b
    return (y * HADAMARD_SCALE).astype(np.float32).reshape(rows, K)


def hadamard_quantize_mxfp4(x):
    """Fused activation transform: Hadamard-32 rotation, then the MXFP4 block quantiser."""
    return quantize_mxfp4(hadamard32(x))


def mxfp4_gemm_ref(a_packed, a_scales, b_packed, b_scales):
    """fp32 product of the dequantised operands: A (M, K/2), B (N, K/2) -> (M, N)."""
    a = dequantize_mxfp4(a_packed, a_scales).astype(np.float32)
    b = dequantize_mxfp4(b_packed, b_scales).astype(np.float32)
    import torch
    return torch.matmul(torch.from_numpy(a), torch.from_numpy(b).T).numpy()
