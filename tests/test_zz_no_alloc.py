"""The stream-K entry point that brings its own scratch memory (for callers that may not allocate on the device: all of
HBM already belongs to their arena, or cudaMalloc's device-wide synchronisation is off limits on their latency path).

Called straight through the C ABI and compared, twice in a row, with the regular entry point (tb_gemm with a caller
workspace) and with the CPU oracle on the same inputs: the second call finds the built-in array holding the first call's
flags and partial tiles. Tolerance as in the other GEMM tests: rtol 1e-2 plus 1e-2 of the reference's rms (both entry
points run the same kernel with the same schedule, so their results are expected to be identical).

"Allocates nothing" is checked three ways: torch's allocator sees no request during a call; the driver's free-memory
figure does not move across calls made by a fresh process that never touches the regular entry point; and the library's
sources name no allocator at all (tests/test_abi_symbols.py, runs without a GPU)."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from tests._util import assert_close_to_oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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
        assert_close_to_oracle(out, a, b, what=f"built-in scratch, call {call}")
    del before


def test_launch_without_a_split_tile_is_never_refused():
    """A grid that divides the tile count leaves no tile to split: no partial tile is written, so the 10 MB limit does not
    apply however large programs x tile is."""
    from tritonblas_b200 import _lib
    lib = _lib.lib
    m, n, k = 1024, 9472, 512                       # 4 x 37 = 148 tiles of 256 x 256 on 74 CTA pairs: two tiles each
    gen = torch.Generator().manual_seed(5)
    a = torch.randn(m, k, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(n, k, generator=gen).to(torch.bfloat16).cuda().T
    c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    prob = _lib.Problem(m=m, n=n, k=k, a_dtype=_lib.BF16, b_dtype=_lib.BF16, c_dtype=_lib.BF16, streamk=1, device=0)
    cfg = _lib.Config()
    assert lib.tb_select(ctypes.byref(prob), ctypes.byref(cfg)) == 0
    cfg.cta_pair, cfg.block_m, cfg.block_n, cfg.sk_grid = 2, 256, 256, 74
    assert 74 * 2 * 128 * 256 * 4 > 10 * 1024 * 1024
    rc = lib.tb_gemm_streamk_builtin(ctypes.byref(_args(_lib, a, b, c, True)), ctypes.byref(cfg), _lib.current_stream_ptr(), None)
    _lib.check(rc, "tb_gemm_streamk_builtin")
    assert_close_to_oracle(c, a, b, rows=[0, 255, 256, 1023], what="whole-tile launch on built-in scratch")


def test_rejects_what_only_the_regular_entry_point_offers():
    from tritonblas_b200 import _lib
    lib = _lib.lib
    a = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    c = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    for field, value in (("epilogue_op", 1), ("num_c_copies", 1), ("num_groups", 2)):
        g = _args(_lib, a, a.T, c, True)
        setattr(g, field, value)
        assert lib.tb_gemm_streamk_builtin(ctypes.byref(g), None, _lib.current_stream_ptr(), None) == 2, field


_FRESH = r"""
import ctypes, os, sys, torch
sys.path.insert(0, os.environ["TB_ROOT"])
from tritonblas_b200 import _lib
from oracle import gemm_oracle
lib = _lib.lib
torch.cuda.set_device(0)
m, n, k = 384, 640, 4096
gen = torch.Generator().manual_seed(1)
a = torch.randn(m, k, generator=gen).to(torch.bfloat16).cuda()
b = torch.randn(n, k, generator=gen).to(torch.bfloat16).cuda().T
outs = [torch.empty(m, n, dtype=torch.bfloat16, device="cuda") for _ in range(3)]
def call(out):
    g = _lib.GemmArgs()
    g.m, g.n, g.k = m, n, k
    g.a_dtype = g.b_dtype = g.c_dtype = _lib.BF16
    g.a, g.a_stride_m, g.a_stride_k = a.data_ptr(), a.stride(0), a.stride(1)
    g.b, g.b_stride_k, g.b_stride_n = b.data_ptr(), b.stride(0), b.stride(1)
    g.c, g.c_stride_m, g.c_stride_n = out.data_ptr(), out.stride(0), out.stride(1)
    g.allow_tf32, g.streamk, g.sk_grid = 1, 1, 37
    rc = lib.tb_gemm_streamk_builtin(ctypes.byref(g), None, _lib.current_stream_ptr(), None)
    assert rc == 0, rc
    torch.cuda.synchronize()
# the first call does the per-device set-up (symbol addresses; the driver loads the kernel image on first use)
call(outs[0])
free0, _ = torch.cuda.mem_get_info()
call(outs[1]); call(outs[2])
free1, _ = torch.cuda.mem_get_info()
assert free1 == free0, ("device memory moved across calls", free0, free1)
ref = gemm_oracle.gemm_ref_f32(a, b)
rms = ref.pow(2).mean().sqrt().item()
for o in outs:
    err = (o.float().cpu() - ref).abs()
    assert bool((err <= 1e-2 * ref.abs() + 1e-2 * rms).all()), err.max().item()
print("fresh process ok")
"""


def test_fresh_process_that_only_uses_the_built_in_entry_point():
    """No call of the regular entry point (or anything else of the library) comes first, so whatever set-up the built-in
    path needs, it does itself; the driver's free-memory figure is the same before and after two further calls."""
    env = dict(os.environ, TB_ROOT=ROOT)
    res = subprocess.run([sys.executable, "-c", _FRESH], env=env, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "fresh process ok" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]


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
