"""fp32-accumulate GEMM oracle (test infrastructure; see oracle/__init__.py).

Follows the reference's epilogue contract: accumulate in fp32, then scale by a_scale[:, None], then by
b_scale[None, :], then add bias broadcast over rows, then one cast to the output type
(include/tritonblas/kernels/stages/matrix_view.py:147-208,263-301; tests/test_matmul_a8w8_lt.py:11-38).
"""
import torch


def gemm_ref(a, b, out_dtype=None, a_scale=None, b_scale=None, bias=None):
    """C = cast(((A.float() @ B.float()) * a_scale[:, None]) * b_scale[None, :] + bias[None, :]) on the CPU."""
    out_dtype = out_dtype or a.dtype
    if a.dtype == torch.int8:
        # integer operands accumulate exactly in int32 on the tensor cores (reference: acc_dtype int32 for int8,
        # kernels/persistent_gemm.py:75); fp64 holds those sums exactly, then the epilogue runs in fp32
        acc = torch.matmul(a.detach().cpu().to(torch.float64), b.detach().cpu().to(torch.float64)).to(torch.float32)
    else:
        acc = torch.matmul(a.detach().cpu().to(torch.float32), b.detach().cpu().to(torch.float32))
    if a_scale is not None:
        acc = acc * a_scale.detach().cpu().to(torch.float32).reshape(-1, 1)
    if b_scale is not None:
        acc = acc * b_scale.detach().cpu().to(torch.float32).reshape(1, -1)
    if bias is not None:
        acc = acc + bias.detach().cpu().to(torch.float32).reshape(1, -1)
    if out_dtype == torch.float8_e4m3fn:
        acc = acc.clamp(-448.0, 448.0)  # saturating cast, tests/test_matmul_a8w8_lt.py:27-32
    if out_dtype == torch.int8:
        acc = acc.round().clamp(-128.0, 127.0)
    return acc.to(out_dtype)


def gemm_ref_f32(a, b, a_scale=None, b_scale=None, bias=None):
    """Same as gemm_ref but left in fp32 (for error measurement before the output cast)."""
    return gemm_ref(a, b, torch.float32, a_scale, b_scale, bias)


def quantize_per_channel_ref(x, dtype, axis):
    """Per-row (axis=1) or per-column (axis=0) symmetric quantisation to fp8/int8 as the reference fixture does
    (include/tritonblas/utils.py:340-377): scale = clamp(amax, 1e-8) / dtype_max, q = (x * (1/scale)).to(dtype).

    The fixture runs where its input lives, which in the reference's tests is the GPU, and there torch divides a tensor
    by a Python scalar as a multiplication by the scalar's fp32 reciprocal; this restatement does the same so that it
    reproduces the reference's scales bit for bit (a true division differs by one ulp for some rows)."""
    xf = x.detach().cpu().to(torch.float32)
    if dtype.is_floating_point:
        qmax = torch.finfo(dtype).max
    else:
        qmax = torch.iinfo(dtype).max
    amax = xf.abs().amax(dim=axis, keepdim=True).clamp(min=1e-8)
    scale = amax * (torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(qmax), dtype=torch.float32))
    q = xf * (1.0 / scale)
    if not dtype.is_floating_point:
        q = q.round().clamp(-qmax, qmax)
    return q.to(dtype), scale.reshape(-1).to(torch.float32)


def grouped_gemm_ref(x, weights, group_offsets, out_dtype=None):
    """Grouped (MoE) GEMM: rows [group_offsets[e], group_offsets[e+1]) of x times weights[e] (K, N) -> out rows.

    No reference implementation exists; semantics = the dense contract applied per expert (fp32 accumulate, one cast).
    """
    out_dtype = out_dtype or x.dtype
    xf = x.detach().cpu().to(torch.float32)
    E = weights.shape[0]
    out = torch.zeros(x.shape[0], weights.shape[2], dtype=torch.float32)
    for e in range(E):
        lo, hi = int(group_offsets[e]), int(group_offsets[e + 1])
        if hi > lo:
            out[lo:hi] = xf[lo:hi] @ weights[e].detach().cpu().to(torch.float32)
    return out.to(out_dtype)
