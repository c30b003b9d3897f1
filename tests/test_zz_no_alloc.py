"""The stream-K entry point that brings its own scratch memory (for callers that may not allocate on the device: all of
HBM already belongs to their arena, or cudaMalloc's device-wide synchronisation is off limits on their latency path).

Called straight through the C ABI and compared with the regular entry point (tb_gemm with a caller workspace) on the same
inputs, twice in a row: the second call finds the built-in array holding the first call's flags and partial tiles.
Tolerance as in the other GEMM tests: rtol 1e-2 plus 1e-2 of the reference's rms (both entry points run the same kernel
with the same schedule, so the results are expected to be identical)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(lib_mod, a, b, c, streamk, workspace=None, epoch=0, sk_grid=0):
    g = lib_mod.GemmArgs()
    g.m, g.n, g.k = a.shape[0], b.shape[1], a.shape[1]
    g.a_dtype = g.b_dtype = lib_mod.DTYPE_CODE[a.dtype]
    g.c_dtype = lib_mod.DTYPE_CODE[c.dtype]
    g.a, g.a_stride_m, g.a_stride_k = a.data_ptr(), a.stride(0), a.stride(1)
    g.b, g.b_stride_k, g.b_stride_n = b.data_ptr(), b.stride(0), b.stride(1)
    g.c, g.c_stride_m, g.c_stride_n = c.data_ptr(), c.stride(0), c.stride(1)
    g.allow_tf32, g.streamk, g.sk_grid = 1, int(streamk), sk_grid
    if workspace is not None:
        g.workspace, g.workspace_bytes, g.epoch = workspace.data_ptr(), workspace.numel(), epoch
    return g


@pytest.mark.parametrize("m,n,k,sk_grid", [(16, 4096, 2048, 0), (384, 640, 4096, 37), (128, 256, 8192, 148)])
def test_builtin_scratch_entry_point_matches_workspace_entry_point(m, n, k, sk_grid):
    from tritonblas_b200 import _lib
    lib = _lib.lib
    gen = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=gen).to(torch.bfloat16).cuda().T          # K-contiguous B
    stream = _lib.current_stream_ptr()
    # regular entry point: caller-owned workspace, library's own configuration for a stream-K launch
    prob = _lib.Problem(m=m, n=n, k=k, a_dtype=_lib.BF16, b_dtype=_lib.BF16, c_dtype=_lib.BF16, streamk=1, device=0)
    cfg = _lib.Config()
    assert lib.tb_select(ctypes.byref(prob), ctypes.byref(cfg)) == 0
    ws = torch.zeros(int(lib.tb_gemm_workspace_bytes(ctypes.byref(cfg), sk_grid)), dtype=torch.uint8, device="cuda")
    ref = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    _lib.check(lib.tb_gemm(ctypes.byref(_args(_lib, a, b, ref, True, ws, 1, sk_grid)), ctypes.byref(cfg), stream), "tb_gemm")
    rms = ref.float().pow(2).mean().sqrt()
    before = torch.cuda.memory_allocated()
    for call in range(2):
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        allocated = torch.cuda.memory_allocated()
        prev = ctypes.c_int32(-1)
        rc = lib.tb_gemm_streamk_builtin(ctypes.byref(_args(_lib, a, b, out, True, None, 0, sk_grid)), ctypes.byref(cfg),
                                         stream, ctypes.byref(prev))
        _lib.check(rc, "tb_gemm_streamk_builtin")
        assert prev.value == 0, f"call {call}: an earlier launch recorded device failure {prev.value}"
        assert torch.cuda.memory_allocated() == allocated          # nothing came from torch's allocator
        torch.cuda.synchronize()
        err = (out.float() - ref.float()).abs()
        assert torch.isfinite(out.float()).all(), f"call {call}"
        assert (err <= 1e-2 * ref.float().abs() + 1e-2 * rms).all(), f"call {call}: max err {err.max().item()}"
    del before


def test_builtin_scratch_rejects_oversized_launch():
    from tritonblas_b200 import _lib
    lib = _lib.lib
    m, n, k = 512, 8192, 4096
    a = torch.zeros(m, k, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(n, k, dtype=torch.bfloat16, device="cuda").T
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    prob = _lib.Problem(m=m, n=n, k=k, a_dtype=_lib.BF16, b_dtype=_lib.BF16, c_dtype=_lib.BF16, streamk=1, device=0)
    cfg = _lib.Config()
    assert lib.tb_select(ctypes.byref(prob), ctypes.byref(cfg)) == 0
    need = (cfg.sk_grid * (2 if cfg.cta_pair == 2 else 1)) * 128 * cfg.block_n * 4
    rc = lib.tb_gemm_streamk_builtin(ctypes.byref(_args(_lib, a, b, c, True)), ctypes.byref(cfg), _lib.current_stream_ptr(), None)
    if need > 10 * 1024 * 1024:
        assert rc == 4 and b"built-in stream-K scratch" in lib.tb_last_cuda_error()
    else:
        assert rc == 0
