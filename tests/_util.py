"""Shared helpers for the GPU parity tests."""
import math

import torch

from oracle import gemm_oracle


def make_operands(m, n, k, dtype, trans_a, trans_b, seed=42, scale=1.0, device="cuda"):
    """Seeded A (m,k) and B (k,n) in the layout the reference's fixture produces
    (include/tritonblas/utils.py:390-538): "T" = K contiguous, "N" = stored transposed and passed as a .T view.
    A uses `seed`, B uses `seed + 10000`."""
    ga = torch.Generator().manual_seed(seed)
    gb = torch.Generator().manual_seed(seed + 10000)
    a = (torch.randn(m, k, generator=ga) * scale)
    b = (torch.randn(k, n, generator=gb) * scale)
    a = a.to(dtype).to(device)
    b = b.to(dtype).to(device)
    if trans_a == "N":
        a = a.T.contiguous().T          # M contiguous
    if trans_b == "T":
        b = b.T.contiguous().T          # K contiguous
    else:
        b = b.contiguous()              # N contiguous
    return a, b


def assert_close_to_oracle(c, a, b, rtol=1e-2, a_scale=None, b_scale=None, bias=None, rows=None, what=""):
    """|c - ref| <= rtol * |ref| + rtol * rms(ref), ref = fp32-accumulate CPU product (optionally on sampled rows)."""
    if rows is not None:
        idx = torch.as_tensor(rows, device=a.device)
        a = a[idx]
        c = c[idx]
        if a_scale is not None:
            a_scale = a_scale[idx]
    ref = gemm_oracle.gemm_ref_f32(a, b, a_scale, b_scale, bias)
    got = c.detach().cpu().to(torch.float32)
    rms = ref.pow(2).mean().sqrt().item()
    err = (got - ref).abs()
    bound = rtol * ref.abs() + rtol * max(rms, 1e-30)
    bad = err > bound
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} elements off; max err {err.max().item():.4g}, "
                           f"rms(ref) {rms:.4g}, first bad {bad.nonzero()[0].tolist()}")
    assert torch.isfinite(got).all(), what
