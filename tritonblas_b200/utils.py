"""Input generation, quantisers and decoders with the names the reference exposes in include/tritonblas/utils.py.

The MXFP4 quantisers run hand-written CUDA kernels through the C ABI; the per-channel FP8/INT8 quantiser and the
decoders are torch-op fixtures, as they are in the reference.
"""
import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple, Union

import torch

from . import _lib

_STR2DTYPE = {"fp16": torch.float16, "float16": torch.float16, "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
              "fp32": torch.float32, "float32": torch.float32, "fp8": torch.float8_e4m3fn,
              "fp8e4m3": torch.float8_e4m3fn, "float8_e4m3fn": torch.float8_e4m3fn, "fp8e5m2": torch.float8_e5m2,
              "float8_e5m2": torch.float8_e5m2, "int8": torch.int8, "uint8": torch.uint8}


def _ensure_dtype(dt):
    if isinstance(dt, torch.dtype):
        return dt
    key = str(dt).lower().replace("torch.", "")
    if key not in _STR2DTYPE:
        raise ValueError(f"Unsupported dtype: {dt}")
    return _STR2DTYPE[key]


def _is_float8_like(dt):
    return dt in (torch.float8_e4m3fn, torch.float8_e5m2)


def _is_int8(dt):
    return dt == torch.int8


@dataclass
class MatmulInputs:
    """What generate_matmul_inputs returns (reference: utils.py:200-262)."""
    A: torch.Tensor
    B: torch.Tensor
    C: torch.Tensor
    bias: torch.Tensor
    scaleA: Optional[torch.Tensor] = None
    scaleB: Optional[torch.Tensor] = None

    @property
    def is_quantized(self):
        return self.scaleA is not None and self.scaleB is not None

    @property
    def is_fp4(self):
        return self.is_quantized and self.scaleA.ndim == 2 and self.scaleB.ndim == 2


def matmul_input_gen(size, dtype, init_type, *, quantize=None, min_scale=1e-8, device="cuda"):
    """A tensor of `size` initialised by `init_type` ("randn", "hpl", "trig_float", "zeros"); with `quantize` it is
    scaled per row to FP8/INT8 and (q, scale[(M, 1)]) is returned (reference: utils.py:264-337)."""
    dtype = _ensure_dtype(dtype)
    M, N = size
    if init_type == "hpl":
        base = torch.empty(size, device=device, dtype=torch.float32).uniform_(-0.5, 0.5)
    elif init_type == "trig_float":
        base = torch.arange(0, M * N, device=device, dtype=torch.float32).reshape(M, N).sin()
    elif init_type == "zeros":
        base = torch.zeros(size, dtype=torch.float32, device=device)
    elif init_type == "randn":
        base = torch.randn(size, dtype=torch.float32, device=device)
    else:
        raise ValueError(f"Unsupported init_type: {init_type}")
    mode = quantize
    if mode == "auto":
        mode = "fp8" if _is_float8_like(dtype) else "int8" if _is_int8(dtype) else None
    if mode is None:
        return base.to(dtype)
    amax = base.abs().amax(dim=1, keepdim=True).clamp(min=min_scale)
    if mode == "fp8":
        scale = amax / torch.finfo(dtype).max
        return (base / scale).to(dtype), scale.to(torch.float32)
    if mode == "int8":
        scale = amax / 127.0
        return torch.round(base / scale).clamp_(-127.0, 127.0).to(torch.int8), scale.to(torch.float32)
    raise ValueError(f"Unsupported quantize mode: {mode}")


def quantize_tensor_per_channel(tensor, target_dtype, axis, *, min_scale=1e-8):
    """Symmetric per-channel quantisation along `axis`: scale = clamp(amax, min_scale) / dtype_max,
    q = (x * (1/scale)).to(dtype); returns (q, scale squeezed to 1-D fp32) (reference: utils.py:340-377)."""
    dtype = _ensure_dtype(target_dtype)
    if not (_is_float8_like(dtype) or _is_int8(dtype)):
        raise ValueError(f"Unsupported quantized dtype: {dtype}")
    base = tensor.to(torch.float32)
    amax = base.abs().amax(dim=axis, keepdim=True).clamp(min=min_scale)
    qmax = torch.finfo(dtype).max if _is_float8_like(dtype) else 127.0
    scale = amax / qmax
    q = base * (1.0 / scale)
    if _is_int8(dtype):
        q = torch.round(q).clamp_(-qmax, qmax)
    return q.to(dtype), scale.squeeze(axis).to(torch.float32)


class Mxfp4ScaleAtoms:
    """e8m0 scales of a (rows, k) operand in the arrangement the block-scaled tensor-core copy consumes:
    [ceil(rows/128)][ceil(k/128)][512 bytes], byte of (row r, K block j) at (r % 32) * 16 + ((r % 128) / 32) * 4 + j % 4
    inside its atom, padding = 127. matmul_fp4 accepts this in place of the row-major (rows, k/32) tensor and then skips
    its own re-arrangement pass."""

    def __init__(self, data, rows, k):
        self.data, self.rows, self.k = data, int(rows), int(k)

    @property
    def shape(self):
        return (self.rows, self.k // 32)

    def to_row_major(self):
        """Back to the (rows, k/32) layout of the reference API (a torch gather; for tests and debugging)."""
        k_atoms = -(-self.k // 128)
        r = torch.arange(self.rows, device=self.data.device).view(-1, 1)
        j = torch.arange(self.k // 32, device=self.data.device).view(1, -1)
        off = ((r // 128) * k_atoms + j // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4
        return self.data[off]


def mxfp4_scales_to_atoms(scales, k=None):
    """Re-arrange row-major e8m0 scales (rows, k/32) into :class:`Mxfp4ScaleAtoms` (one small CUDA kernel)."""
    if isinstance(scales, Mxfp4ScaleAtoms):
        return scales
    scales = scales.view(torch.uint8)
    if scales.stride(1) != 1:
        scales = scales.contiguous()
    rows, kblocks = scales.shape
    k = kblocks * 32 if k is None else k
    nbytes = int(_lib.lib.tb_mxfp4_atoms_bytes(rows, k))
    atoms = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=scales.device)
    if rows and kblocks:
        with torch.cuda.device(scales.device):
            rc = _lib.lib.tb_mxfp4_scales_to_atoms(ctypes.c_void_p(scales.data_ptr()), scales.stride(0), rows, k,
                                                   ctypes.c_void_p(atoms.data_ptr()), _lib.current_stream_ptr(scales.device))
        _lib.check(rc, "tb_mxfp4_scales_to_atoms")
    return Mxfp4ScaleAtoms(atoms, rows, k)


def quantize_fp8_rows(x: torch.Tensor):
    """Per-row FP8 e4m3 quantisation on the GPU (one CUDA kernel): returns (q (rows, K) float8_e4m3fn, scale (rows,)
    fp32) with scale = max(amax, 1e-8) / 448 and q = (x * (1 / scale)).to(e4m3), the arithmetic of
    quantize_tensor_per_channel(x, float8_e4m3fn, axis=1). Use it on activations (per token) and on weights stored
    (N, K) (per output channel)."""
    assert x.ndim == 2 and x.shape[1] % 8 == 0, "x must be (rows, K) with K a multiple of 8"
    if not x.is_cuda:
        raise RuntimeError("the FP8 quantiser runs on CUDA tensors only (no CPU path)")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported input dtype: {x.dtype}")
    if x.stride(1) != 1 or (x.stride(0) * 2) % 16 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    if x.numel():
        with torch.cuda.device(x.device):
            rc = _lib.lib.tb_fp8_quant_rows(ctypes.c_void_p(x.data_ptr()), _lib.DTYPE_CODE[x.dtype], x.shape[0], x.shape[1],
                                            x.stride(0), ctypes.c_void_p(q.data_ptr()), q.stride(0),
                                            ctypes.c_void_p(scale.data_ptr()), _lib.current_stream_ptr(x.device))
        _lib.check(rc, "tb_fp8_quant_rows")
    return q, scale


def _mxfp4_quant(x, hadamard, scale_atoms=False, out=None):
    assert x.ndim == 2, "Input must be 2D tensor"
    M, N = x.shape
    assert N % 32 == 0, f"N ({N}) must be divisible by 32"
    if not x.is_cuda:
        raise RuntimeError("the MXFP4 quantiser runs on CUDA tensors only (no CPU path)")
    if x.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError(f"Unsupported input dtype: {x.dtype}")
    es = x.element_size()
    if x.stride(1) != 1 or (x.stride(0) * es) % 16 != 0 or x.data_ptr() % 16 != 0:
        x = x.contiguous()
    atoms = scales = None
    if out is not None:
        # the (codes, scales) pair of an earlier call with the same shape and flags: nothing is allocated or filled
        codes, second = out
        assert tuple(codes.shape) == (M, N // 2) and codes.dtype == torch.uint8 and codes.device == x.device
        if scale_atoms:
            assert isinstance(second, Mxfp4ScaleAtoms) and (second.rows, second.k) == (M, N)
            atoms = second.data
        else:
            assert tuple(second.shape) == (M, N // 32)
            scales = second
    else:
        codes = torch.empty((M, N // 2), dtype=torch.uint8, device=x.device)
        if scale_atoms:   # padding rows and blocks of the atom layout hold 127 (scale 1.0); the kernel writes the rest
            atoms = torch.full((max(int(_lib.lib.tb_mxfp4_atoms_bytes(M, N)), 16),), 127, dtype=torch.uint8, device=x.device)
        else:
            scales = torch.empty((M, N // 32), dtype=torch.uint8, device=x.device)
    if M == 0 or N == 0:
        return (codes, Mxfp4ScaleAtoms(atoms, M, N)) if scale_atoms else (codes, scales)
    with torch.cuda.device(x.device):
        rc = _lib.lib.tb_mxfp4_quant_atoms(ctypes.c_void_p(x.data_ptr()), _lib.DTYPE_CODE[x.dtype], M, N, x.stride(0),
                                           ctypes.c_void_p(codes.data_ptr()), codes.stride(0),
                                           ctypes.c_void_p(scales.data_ptr() if scales is not None else 0),
                                           scales.stride(0) if scales is not None else N // 32,
                                           ctypes.c_void_p(atoms.data_ptr()) if scale_atoms else ctypes.c_void_p(0),
                                           int(hadamard), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "tb_mxfp4_quant")
    if scale_atoms:
        return codes, Mxfp4ScaleAtoms(atoms, M, N)
    return codes, scales


def dynamic_mxfp4_quant(x: torch.Tensor, scale_atoms: bool = False, out=None):
    """x (M, N) -> packed e2m1 codes (M, N/2) uint8 and e8m0 scales (M, N/32) uint8, one scale per 32 contiguous
    elements; bit-identical to the reference quantiser (utils.py:742-789). With ``scale_atoms`` the scales come back as
    :class:`Mxfp4ScaleAtoms`, ready for matmul_fp4 without a re-arrangement pass. ``out``: the pair an earlier call with
    the same shape and flags returned; it is overwritten and returned (no allocation, no fill: a steady-state step is
    then one kernel)."""
    return _mxfp4_quant(x, False, scale_atoms, out)


def hadamard_mxfp4_quant(x: torch.Tensor, scale_atoms: bool = False, out=None):
    """Fused activation transform: rotate every 32-element block by H32/sqrt(32), then quantise to MXFP4.
    Apply it to both operands' K blocks: (A H)(B H)^T = A B^T because H is orthonormal and symmetric. ``out`` as in
    :func:`dynamic_mxfp4_quant`."""
    return _mxfp4_quant(x, True, scale_atoms, out)


_E2M1_TABLE = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def mxfp4_to_f32(x: torch.Tensor) -> torch.Tensor:
    """Unpack e2m1 pairs (low nibble first) to fp32 (reference: utils.py:547-607)."""
    if hasattr(torch, "float4_e2m1fn_x2") and x.dtype == torch.float4_e2m1fn_x2:
        x = x.view(torch.uint8)
    lut = torch.tensor(_E2M1_TABLE, dtype=torch.float32, device=x.device)
    lo = lut[(x & 0xF).long()]
    hi = lut[(x >> 4).long()]
    return torch.stack((lo, hi), dim=-1).reshape(*x.shape[:-1], x.shape[-1] * 2)


def e8m0_to_f32(scale_e8m0: torch.Tensor) -> torch.Tensor:
    """Exponent bytes to fp32 2^(s-127); 0 decodes to the bit pattern 0x00400000, 255 to NaN
    (reference: utils.py:610-643)."""
    s = scale_e8m0.view(torch.uint8)
    bits = s.to(torch.int32) << 23
    bits = torch.where(s == 0, torch.full_like(bits, 0x00400000), bits)
    bits = torch.where(s == 0xFF, torch.full_like(bits, 0x7F800001), bits)
    return bits.view(torch.float32)


def generate_matmul_inputs(m, n, k, in_dtype=None, out_dtype=torch.float16, transA="T", transB="T", init_type="randn",
                           *, device="cuda", quantize_mode="auto", dtype_a=None, dtype_b=None, seed=None) -> MatmulInputs:
    """A (m, k), B (k, n), C (m, n), bias (m,) and, for fp8/int8/"fp4" inputs, their scales (reference:
    utils.py:390-538). "T" keeps the matrix as generated; "N" generates the transposed shape and passes a .T view.
    A is seeded with `seed`, B with `seed + 10000`."""
    dtype_a = in_dtype if dtype_a is None else dtype_a
    dtype_b = in_dtype if dtype_b is None else dtype_b
    if dtype_a is None or dtype_b is None:
        raise ValueError("Either in_dtype or dtype_a/dtype_b must be provided")
    fp4_a = isinstance(dtype_a, str) and dtype_a.lower() == "fp4"
    fp4_b = isinstance(dtype_b, str) and dtype_b.lower() == "fp4"
    dtype_a = torch.uint8 if fp4_a else _ensure_dtype(dtype_a)
    dtype_b = torch.uint8 if fp4_b else _ensure_dtype(dtype_b)
    out_dtype = _ensure_dtype(out_dtype)
    if transA not in ("T", "N") or transB not in ("T", "N"):
        raise ValueError("transA/transB must be 'T' or 'N'")

    def init(shape, s):
        if s is not None:
            torch.manual_seed(s)
            if str(device).startswith("cuda"):
                torch.cuda.manual_seed(s)
        return matmul_input_gen(shape, torch.float32, init_type, device=device)

    A = init((m, k), seed) if transA == "T" else init((k, m), seed).T
    b_seed = seed + 10000 if seed is not None else None
    B = init((k, n), b_seed) if transB == "T" else init((n, k), b_seed).T
    scaleA = scaleB = None
    if fp4_a or fp4_b:
        if k % 32 != 0:
            raise ValueError(f"For FP4 quantization, K must be divisible by 32, got K={k}")
        A, scaleA = dynamic_mxfp4_quant(A.contiguous())            # (m, k/2), (m, k/32)
        Bq, scaleB = dynamic_mxfp4_quant(B.T.contiguous())          # (n, k/2), (n, k/32)
        B = Bq.T                                                     # (k/2, n) view, K contiguous
    else:
        quant_a = quantize_mode in ("fp8", "int8") or (quantize_mode == "auto" and (_is_float8_like(dtype_a) or _is_int8(dtype_a)))
        quant_b = quantize_mode in ("fp8", "int8") or (quantize_mode == "auto" and (_is_float8_like(dtype_b) or _is_int8(dtype_b)))
        if quant_a:
            A, scaleA = quantize_tensor_per_channel(A, dtype_a, axis=1)
        else:
            A = A.to(dtype_a)
        if quant_b:
            B, scaleB = quantize_tensor_per_channel(B, dtype_b, axis=0)
        else:
            B = B.to(dtype_b)
    C = torch.zeros((m, n), device=device, dtype=out_dtype)
    bias = torch.zeros((m,), device=device, dtype=out_dtype)
    return MatmulInputs(A=A, B=B, C=C, bias=bias, scaleA=scaleA, scaleB=scaleB)
