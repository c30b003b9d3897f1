"""Host API of the GEMM family: same names, argument order and error behaviour as the reference's
include/tritonblas/matmul.py, implemented as thin marshalling over the C ABI (tb_gemm and friends).

No kernel is written here and nothing falls back to torch: a missing library or an unsupported request raises.
"""
import ctypes
from typing import Optional

import torch

from . import _lib
from .config import MatmulConfig, matmul_preamble, workspace_bytes
from .origami import OrigamiMatmulSelector

# Per-device stream-K workspace used when the caller passes no MatmulConfig; like the reference's module-level
# locks/P buffers (matmul.py:20-26) it serves one stream at a time.
_global_workspaces = {}


class _GlobalWorkspace:
    def __init__(self, device, nbytes):
        self.workspace = torch.zeros(nbytes, device=device, dtype=torch.uint8)
        self.epoch = 0

    def next_epoch(self):
        self.epoch = (self.epoch % 0xFFFFFFF0) + 1
        if self.epoch == 1:
            self.workspace[:4096].zero_()
        return self.epoch


_global_tile_counters = {}


def _tile_counter_for(device):
    """Two zeroed words per device for dynamically scheduled launches that bring no MatmulConfig."""
    key = (device.type, device.index)
    buf = _global_tile_counters.get(key)
    if buf is None:
        buf = torch.zeros(64, device=device, dtype=torch.int32)
        _global_tile_counters[key] = buf
    return buf


def _reset_tile_counters():
    """A launch that gave up mid-way leaves its counter words non-zero; zero them before the next dynamic launch."""
    for buf in _global_tile_counters.values():
        buf.zero_()


_lib._failure_hooks.append(_reset_tile_counters)


def _workspace_for(device, nbytes):
    key = (device.type, device.index)
    ws = _global_workspaces.get(key)
    if ws is None or ws.workspace.numel() < nbytes:
        ws = _GlobalWorkspace(device, max(nbytes, 4096 + 148 * 128 * 256 * 4))
        _global_workspaces[key] = ws
    return ws


def _make_matmul_selector(M, N, K, a_dtype, b_dtype, c_dtype, device, mx_block_size=0, streamk=False, num_stages=2,
                          a_mn_major=False, b_mn_major=False, max_halves=0):
    return OrigamiMatmulSelector(M, N, K, a_dtype, b_dtype, c_dtype, device, mx_block_size=mx_block_size,
                                 streamk=streamk, num_stages=num_stages, a_mn_major=a_mn_major, b_mn_major=b_mn_major,
                                 max_halves=max_halves)


def _unit_stride_2d(t):
    """Kernels take any 2-D view with one unit stride; anything else is materialised row-major."""
    if t.stride(1) == 1 or t.stride(0) == 1:
        return t
    return t.contiguous()


def _is_mn_major(t, contiguous_axis_is_k_index):
    """True when the K axis (index given) of a 2-D operand is NOT its unit-stride axis."""
    other = 1 - contiguous_axis_is_k_index
    if t.stride(contiguous_axis_is_k_index) == 1 or t.shape[contiguous_axis_is_k_index] == 1:
        return False
    return t.stride(other) == 1 or t.shape[other] == 1


def _tma_loadable(t):
    """True when a 2-D operand can be described by a TMA tensor map: 16-byte aligned base and pitch."""
    if t.data_ptr() % 16:
        return False
    pitch_axis = 0 if t.stride(1) == 1 else 1
    return t.shape[pitch_axis] == 1 or (t.stride(pitch_axis) * t.element_size()) % 16 == 0


def _repitch(t):
    """Copy of a 2-D operand with the same logical shape and unit-stride axis, its pitch rounded up to 16 bytes.

    The tensor-core kernels load operands with TMA, which needs a 16-byte aligned base and pitch; operands that miss
    that (K or M/N not a multiple of 8 for 16-bit types, odd views) would otherwise run on the CUDA-core kernel, which
    is ~30x slower on large products. The padding is never read: the tensor map keeps the logical extents.
    """
    per16 = 16 // t.element_size()
    if t.stride(1) == 1:
        rows, cols = t.shape
        buf = torch.empty((rows, -(-cols // per16) * per16), dtype=t.dtype, device=t.device)[:, :cols]
    else:
        rows, cols = t.shape
        buf = torch.empty((cols, -(-rows // per16) * per16), dtype=t.dtype, device=t.device)[:, :rows].T
    buf.copy_(t)
    return buf


# Below this many multiply-adds an unaligned product stays on the CUDA-core kernel (a re-pitch costs two small launches).
_REPITCH_MIN_MACS = 1 << 27


def _strides(t):
    """Element strides with any extent-1 axis given its dense stride (such an axis may carry an arbitrary one)."""
    s0, s1 = t.stride()
    if t.shape[0] == 1 and s1 == 1:
        s0 = t.shape[1]
    if t.shape[1] == 1 and s0 == 1:
        s1 = t.shape[0]
    return s0, s1


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _gemm(a, b, c, selector, config=None, bias=None, a_scale=None, b_scale=None, streamk=False, sk_grid=None,
          c_copies=None, work_stealing=False, c_copies_tail_stream=None, c_copies_tail_fraction=0.0, static_b=False,
          c_copies_tile_limit=0):
    assert a.shape[1] == b.shape[0], "Incompatible Dimensions"
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise RuntimeError("tritonblas_b200 runs on CUDA tensors only (no CPU path)")
    M, K = a.shape
    _, N = b.shape
    if tuple(c.shape) != (M, N):
        raise RuntimeError(f"output has shape {tuple(c.shape)}, expected {(M, N)}")
    if M == 0 or N == 0:
        return c
    b_in_ptr = b.data_ptr()
    a = _unit_stride_2d(a)
    b = _unit_stride_2d(b)
    if M * N * K >= _REPITCH_MIN_MACS and a.dtype != torch.float32:
        if not _tma_loadable(a):
            a = _repitch(a)
        if not _tma_loadable(b):
            b = _repitch(b)
    a_mn, b_mn = _is_mn_major(a, 1), _is_mn_major(b, 0)
    cfg = selector.config_for(a_mn, b_mn)

    args = _lib.GemmArgs()
    args.m, args.n, args.k = M, N, K
    args.a_dtype, args.b_dtype, args.c_dtype = (_lib.DTYPE_CODE[a.dtype], _lib.DTYPE_CODE[b.dtype], _lib.DTYPE_CODE[c.dtype])
    args.a, (args.a_stride_m, args.a_stride_k) = _ptr(a), _strides(a)
    args.b, (args.b_stride_k, args.b_stride_n) = _ptr(b), _strides(b)
    args.c, (args.c_stride_m, args.c_stride_n) = _ptr(c), _strides(c)
    if a_scale is not None:
        a_scale = a_scale.to(torch.float32).contiguous().view(-1)
        b_scale = b_scale.to(torch.float32).contiguous().view(-1)
        assert a_scale.numel() == M and b_scale.numel() == N, "scale vectors must be (M,) and (N,)"
        args.a_scale, args.b_scale = _ptr(a_scale), _ptr(b_scale)
    if bias is not None:
        assert bias.numel() == N, "bias must have N elements"
        bias = bias.view(-1)
        args.bias, args.bias_stride, args.bias_dtype = _ptr(bias), bias.stride(0), _lib.DTYPE_CODE[bias.dtype]
    if c_copies:
        # raw device addresses of further destinations laid out exactly like c (peer GPUs' buffers)
        ptrs = (ctypes.c_void_p * len(c_copies))(*[int(p) for p in c_copies])
        args.c_copies, args.num_c_copies = ptrs, len(c_copies)
    if c_copies and c_copies_tile_limit > 0:
        args.c_copies_tile_limit = int(c_copies_tile_limit)     # the caller sends the other tiles itself
    tail_first = None
    if c_copies and c_copies_tail_stream is not None and c_copies_tail_fraction > 0 and not streamk and not cfg.swap_ab \
            and c.stride(1) == 1 and (c.stride(0) * c.element_size()) % 16 == 0 and (N * c.element_size()) % 16 == 0 \
            and _tma_loadable(a) and _tma_loadable(b) and (a.dtype != torch.float32 or torch.backends.cuda.matmul.allow_tf32):
        tiles = int(_lib.lib.tb_gemm_tile_count(ctypes.byref(args), ctypes.byref(cfg)))
        first = tiles - int(tiles * min(float(c_copies_tail_fraction), 1.0))
        if 0 <= first < tiles:
            tail_first = first
            if first > 0:
                args.c_copies_tile_limit = first
            else:
                args.num_c_copies = 0       # nothing leaves from the epilogue; the copy kernel sends every tile
    args.allow_tf32 = int(torch.backends.cuda.matmul.allow_tf32)
    if static_b and b.data_ptr() == b_in_ptr:
        args.static_operands = 2    # the caller's own b (not a re-pitched copy made above, which this stream just wrote)
    if config is not None:
        args.wait_timeout_ms, args.debug_flags = int(config.wait_timeout_ms), int(config.debug_flags)
    args.streamk = int(bool(streamk))
    args.sk_grid = int(sk_grid) if sk_grid else 0
    if work_stealing and not streamk:
        # dynamic tile schedule: the kernel leaves the two counter words zeroed, so launches on one stream share them
        counter = config.tile_counter if config is not None else _tile_counter_for(a.device)
        args.tile_counter = _ptr(counter)
    if streamk:
        need = workspace_bytes(cfg, args.sk_grid)
        holder = config if (config is not None and config.workspace.numel() >= need) else _workspace_for(a.device, need)
        args.workspace, args.workspace_bytes = _ptr(holder.workspace), holder.workspace.numel()
        args.epoch = holder.next_epoch()
    if a.device.index is None or a.device.index == torch.cuda.current_device():
        rc = _lib.lib.tb_gemm(ctypes.byref(args), ctypes.byref(cfg), _lib.current_stream_ptr(a.device))
    else:
        with torch.cuda.device(a.device):
            rc = _lib.lib.tb_gemm(ctypes.byref(args), ctypes.byref(cfg), _lib.current_stream_ptr(a.device))
    if rc:
        _lib.check(rc, "tb_gemm")
    if tail_first is not None:
        # the launch's last tiles travel on the side stream, beside whatever the caller enqueues next on this one
        main = torch.cuda.current_stream(a.device)
        c_copies_tail_stream.wait_stream(main)
        args.num_c_copies = len(c_copies)
        with torch.cuda.stream(c_copies_tail_stream):
            rc = _lib.lib.tb_push_c_tiles(ctypes.byref(args), ctypes.byref(cfg), tail_first,
                                          ctypes.c_void_p(c_copies_tail_stream.cuda_stream))
        _lib.check(rc, "tb_push_c_tiles")
    return c


def persistent_matmul_lt(a, b, c, selector, config=None, bias=None, a_scale=None, b_scale=None, quantized=False,
                         work_stealing=False, c_copies=None, c_copies_tail_stream=None, c_copies_tail_fraction=0.0,
                         static_b=False, c_copies_tile_limit=0):
    """Data-parallel persistent GEMM (reference: matmul.py:69-200). ``work_stealing`` selects the dynamic tile schedule
    (tiles taken from a device counter, matmul.py:112-159) instead of the static round-robin. ``c_copies``: device addresses of further buffers laid out like ``c`` (peer GPUs) that the
    epilogue also writes. With ``c_copies_tail_stream`` (a torch.cuda.Stream) and ``c_copies_tail_fraction`` in (0, 1] the
    epilogue sends only the first tiles and the last ``fraction`` of the tiles are copied to the peers by a kernel on that
    stream after the launch, where they overlap whatever is enqueued next on the current stream; the caller waits for that
    stream before the copies are read. ``c_copies_tile_limit`` > 0 alone: the epilogue sends only tiles with a launch-order
    index below it and the caller moves the rest of ``c`` itself. ``static_b``: a promise that nothing still in flight on the stream writes ``b``
    (weights); the kernel may then start reading it while the previous kernel of the stream is still draining."""
    return _gemm(a, b, c, selector, config, bias, a_scale, b_scale, streamk=False, c_copies=c_copies,
                 work_stealing=work_stealing, c_copies_tail_stream=c_copies_tail_stream,
                 c_copies_tail_fraction=c_copies_tail_fraction, static_b=static_b, c_copies_tile_limit=c_copies_tile_limit)


def streamk_matmul_lt(a, b, c, selector, config=None, bias=None, sk_grid=None, a_scale=None, b_scale=None,
                      quantized=False, work_stealing=False, static_b=False):
    """Hybrid stream-K GEMM (reference: matmul.py:202-366). ``static_b``: see persistent_matmul_lt."""
    return _gemm(a, b, c, selector, config, bias, a_scale, b_scale, streamk=True, sk_grid=sk_grid, static_b=static_b)


def matmul_lt(a, b, c, selector, config: Optional[MatmulConfig] = None, enable_streamk=False, work_stealing=False,
              static_b=False):
    assert a.shape[1] == b.shape[0], "Incompatible Dimensions"
    if enable_streamk:
        return streamk_matmul_lt(a, b, c, selector, config, work_stealing=work_stealing, static_b=static_b)
    return persistent_matmul_lt(a, b, c, selector, config, work_stealing=work_stealing, static_b=static_b)


def matmul_a8w8_lt(a, b, a_scale, b_scale, c, selector, config: Optional[MatmulConfig] = None, enable_streamk=False,
                   work_stealing=False, static_b=False):
    assert a.shape[1] == b.shape[0], "Incompatible Dimensions"
    if enable_streamk:
        return streamk_matmul_lt(a, b, c, selector, config, a_scale=a_scale, b_scale=b_scale, quantized=True,
                                 static_b=static_b)
    return persistent_matmul_lt(a, b, c, selector, config, a_scale=a_scale, b_scale=b_scale, quantized=True,
                                work_stealing=work_stealing, static_b=static_b)


_selector_cache = {}


def _selector_for(a, b, c_dtype, streamk):
    """Selector for the convenience entry points (the reference re-runs its selector on every call, matmul.py:407; the
    result only depends on the key below, so it is kept)."""
    M, K = a.shape
    _, N = b.shape
    a_mn = _is_mn_major(_unit_stride_2d(a), 1)
    b_mn = _is_mn_major(_unit_stride_2d(b), 0)
    key = (M, N, K, a.dtype, b.dtype, c_dtype, a.device, bool(streamk), a_mn, b_mn)
    sel = _selector_cache.get(key)
    if sel is None:
        if len(_selector_cache) >= 1024:
            _selector_cache.clear()
        sel = _make_matmul_selector(M, N, K, a.dtype, b.dtype, c_dtype, a.device, streamk=bool(streamk),
                                    a_mn_major=a_mn, b_mn_major=b_mn)
        _selector_cache[key] = sel
    return sel


# ---------------------------------------------------------------------------------------------- custom ops
@torch.library.custom_op("tritonblas::_matmul", mutates_args=())
def _matmul(a: torch.Tensor, b: torch.Tensor, enable_streamk: Optional[bool] = False, sk_grid: Optional[int] = None,
            work_stealing: Optional[bool] = False) -> torch.Tensor:
    assert a.shape[1] == b.shape[0], "Incompatible A-B Dimensions"
    out = a.new_empty(a.shape[0], b.shape[1])
    selector = _selector_for(a, b, out.dtype, enable_streamk)
    if enable_streamk:
        streamk_matmul_lt(a, b, out, selector, None, sk_grid=sk_grid, work_stealing=work_stealing)
    else:
        persistent_matmul_lt(a, b, out, selector, None, work_stealing=work_stealing)
    return out


@_matmul.register_fake
def _(a, b, enable_streamk=False, sk_grid=None, work_stealing=False):
    return a.new_empty(a.shape[0], b.shape[1])


def _setup_context_matmul_backwards(ctx, inputs, output):
    a, b, enable_streamk, sk_grid, work_stealing = inputs
    ctx.save_for_backward(a, b)
    ctx.enable_streamk, ctx.sk_grid, ctx.work_stealing = enable_streamk, sk_grid, work_stealing


def _matmul_backwards(ctx, grad_output):
    # Two more forward GEMMs on materialised transposes, as the reference does (matmul.py:427-444).
    a, b = ctx.saved_tensors
    kw = dict(enable_streamk=ctx.enable_streamk, sk_grid=ctx.sk_grid, work_stealing=ctx.work_stealing)
    g = grad_output.contiguous()
    grad_a = matmul(g, b.T.contiguous(), **kw) if ctx.needs_input_grad[0] else None
    grad_b = matmul(a.T.contiguous(), g, **kw) if ctx.needs_input_grad[1] else None
    return grad_a, grad_b, None, None, None


_matmul.register_autograd(_matmul_backwards, setup_context=_setup_context_matmul_backwards)


@torch.library.custom_op("tritonblas::_matmul_out", mutates_args={"out"})
def _matmul_out(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, enable_streamk: Optional[bool] = False,
                sk_grid: Optional[int] = None, work_stealing: Optional[bool] = False) -> None:
    assert a.shape[1] == b.shape[0], "Incompatible A-B Dimensions"
    selector = _selector_for(a, b, out.dtype, enable_streamk)
    if enable_streamk:
        streamk_matmul_lt(a, b, out, selector, None, sk_grid=sk_grid, work_stealing=work_stealing)
    else:
        persistent_matmul_lt(a, b, out, selector, None, work_stealing=work_stealing)
    return None


def matmul(a, b, out=None, enable_streamk=False, sk_grid=None, work_stealing=False):
    """C = A @ B. Returns the product, or None when ``out`` is given (the result is written into it)."""
    if out is None:
        return _matmul(a, b, enable_streamk, sk_grid, work_stealing)
    if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad or out.requires_grad):
        raise RuntimeError("tritonblas.matmul(): functions with out=... arguments don't support "
                           "automatic differentiation, but one of the arguments requires grad.")
    return _matmul_out(a, b, out, enable_streamk, sk_grid, work_stealing)


def matmul_a8w8(a, b, a_scale, b_scale, c, enable_streamk=False, work_stealing=False, sk_grid=None):
    """C = cast((A8 . B8 in fp32) * a_scale[:, None] * b_scale[None, :]) (reference: matmul.py:498-517, intended
    semantics tests/test_matmul_a8w8_lt.py:11-38)."""
    assert a.shape[1] == b.shape[0], "Incompatible Dimensions"
    selector = _selector_for(a, b, c.dtype, enable_streamk)
    if enable_streamk:
        return streamk_matmul_lt(a, b, c, selector, None, sk_grid=sk_grid, a_scale=a_scale, b_scale=b_scale, quantized=True)
    return persistent_matmul_lt(a, b, c, selector, None, a_scale=a_scale, b_scale=b_scale, quantized=True)


def grouped_matmul(x, w, group_offsets, out=None, a_scale=None, b_scale=None, selector=None, swiglu=False,
                   work_stealing=False, row_index=None, _debug_flags=0):
    """Grouped (MoE) GEMM: out[r] = x[r] @ w[g].T for every row r of group g, rows of group g being
    [group_offsets[g], group_offsets[g+1]).

    x: (rows, K) K-contiguous; w: (G, N, K) contiguous (each expert's weight stored N x K, the K-contiguous fast layout);
    group_offsets: int32 CUDA tensor of G + 1 ascending offsets (it stays on the device: no host synchronisation);
    out: (rows, N), allocated in x.dtype when omitted. The reference has no grouped kernel; per group this is its dense
    contract (fp32 accumulate, one cast). ``selector`` overrides the tile configuration (tuning and tests).

    ``swiglu=True``: w holds [gate | up] projections, (G, 2*F, K); out is (rows, F) = silu(x @ gate.T) * (x @ up.T),
    the activation applied to the fp32 accumulators inside the GEMM's epilogue (F a multiple of 128, more than 128 rows).
    ``work_stealing=True`` selects the dynamic tile schedule.
    ``row_index``: int32 CUDA tensor; grouped row r is then row ``row_index[r]`` of x (a negative entry is a row of zeros)
    and the problem has ``row_index.numel()`` rows: the kernel gathers the rows itself, no gathered copy of x is made.
    """
    assert x.ndim == 2 and w.ndim == 3 and x.shape[1] == w.shape[2], "Incompatible Dimensions"
    if not (x.is_cuda and w.is_cuda and group_offsets.is_cuda):
        raise RuntimeError("tritonblas_b200 runs on CUDA tensors only (no CPU path)")
    rows, K = x.shape
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_cuda and row_index.is_contiguous(), "row_index must be int32 on the GPU"
        rows = row_index.numel()
    G, N, _ = w.shape
    if swiglu:
        assert N % 256 == 0 and a_scale is None, "swiglu needs F = N / 2 to be a multiple of 128 and no scales"
        N //= 2
    assert group_offsets.dtype == torch.int32 and group_offsets.numel() == G + 1, "group_offsets must be int32[G + 1]"
    if out is None:
        out = x.new_empty(rows, N)
    if rows == 0 or N == 0:
        return out
    x = x if x.stride(1) == 1 else x.contiguous()
    w = w if w.is_contiguous() else w.contiguous()
    group_offsets = group_offsets.contiguous()
    # tiles of all groups are pooled over the SMs, so the tile model sees the total row count
    if selector is None:
        # narrow tiles: with many short groups the wide tile's exposed drains outweigh its smaller operand traffic
        selector = _make_matmul_selector(rows, 2 * N if swiglu else N, K, x.dtype, w.dtype, out.dtype, x.device, max_halves=1)
    cfg = selector.config_for(False, False)
    args = _lib.GemmArgs()
    args.m, args.n, args.k = rows, N, K
    args.a_dtype, args.b_dtype, args.c_dtype = (_lib.DTYPE_CODE[x.dtype], _lib.DTYPE_CODE[w.dtype], _lib.DTYPE_CODE[out.dtype])
    args.a, (args.a_stride_m, args.a_stride_k) = _ptr(x), _strides(x)
    args.b, args.b_stride_k, args.b_stride_n = _ptr(w), 1, K
    args.c, (args.c_stride_m, args.c_stride_n) = _ptr(out), _strides(out)
    if a_scale is not None:
        a_scale = a_scale.to(torch.float32).contiguous().view(-1)
        b_scale = b_scale.to(torch.float32).contiguous().view(-1)
        args.a_scale, args.b_scale = _ptr(a_scale), _ptr(b_scale)
    args.allow_tf32 = 1
    args.group_offsets, args.num_groups = _ptr(group_offsets), G
    args.epilogue_op = 1 if swiglu else 0
    if row_index is not None:
        args.a_gather_index, args.a_rows = _ptr(row_index), x.shape[0]
    args.debug_flags = int(_debug_flags)      # measurement switches of the library (tb_gemm_args.debug_flags); 0 in production
    if work_stealing:  # tiles after each program's first come from a device counter (see persistent_matmul_lt)
        args.tile_counter = _ptr(_tile_counter_for(x.device))
    with torch.cuda.device(x.device):
        rc = _lib.lib.tb_grouped_gemm(ctypes.byref(args), ctypes.byref(cfg), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "tb_grouped_gemm")
    return out


def matmul_fp4(a, b, c, a_scales, b_scales, block_m=None, block_n=None, block_k=None, group_size_m=8, num_warps=8,
               num_stages=2):
    """MXFP4 product C = A @ B^T of packed e2m1 operands with e8m0 block-32 scales (reference: matmul.py:519-625).

    a: (M, K/2) uint8, b: (N, K/2) uint8 (two codes per byte, even element in the low nibble), c: (M, N) bf16/fp16/fp32,
    a_scales: (M, K/32) uint8, b_scales: (N, K/32) uint8. ``block_n`` (64, 128 or 192) and
    ``group_size_m`` override the library's choice; block_m, block_k, num_warps and num_stages are accepted for
    signature compatibility (tile height, stage depth and warp roles are fixed by the kernel).
    """
    M, K = a.shape[0], a.shape[1] * 2
    N = b.shape[0]
    assert b.shape[1] * 2 == K, f"Incompatible Dimensions: A has K={K}, B has K={b.shape[1] * 2}"
    assert K % 32 == 0, "K must be a multiple of the MX block size (32)"
    if block_k is not None:
        assert block_k % 64 == 0, "BLOCK_K must be multiple of 64 for FP4"
    if not (a.is_cuda and b.is_cuda and c.is_cuda):
        raise RuntimeError("tritonblas_b200 runs on CUDA tensors only (no CPU path)")
    if hasattr(torch, "float4_e2m1fn_x2"):
        a = a.view(torch.uint8) if a.dtype == torch.float4_e2m1fn_x2 else a
        b = b.view(torch.uint8) if b.dtype == torch.float4_e2m1fn_x2 else b

    def rows_ok(t):
        return t.stride(1) == 1 and t.stride(0) % 16 == 0 and t.data_ptr() % 16 == 0

    a = a if rows_ok(a) else a.contiguous()
    b = b if rows_ok(b) else b.contiguous()
    assert tuple(a_scales.shape) == (M, K // 32) and tuple(b_scales.shape) == (N, K // 32), "scale shapes"
    if M == 0 or N == 0:
        return c
    # The tensor core consumes scales in 128-row x 4-block atoms; row-major scales (the reference layout) are re-arranged
    # by one small kernel each, pre-arranged ones (utils.Mxfp4ScaleAtoms) are used as they are.
    from .utils import mxfp4_scales_to_atoms
    a_atoms = mxfp4_scales_to_atoms(a_scales, K)
    b_atoms = mxfp4_scales_to_atoms(b_scales, K)
    args = _lib.Mxfp4Args()
    args.m, args.n, args.k = M, N, K
    args.a, args.a_row_stride = _ptr(a), a.stride(0)
    args.b, args.b_row_stride = _ptr(b), b.stride(0)
    args.c, (args.c_stride_m, args.c_stride_n), args.c_dtype = _ptr(c), _strides(c), _lib.DTYPE_CODE[c.dtype]
    args.a_scales, args.b_scales, args.scales_in_atoms = _ptr(a_atoms.data), _ptr(b_atoms.data), 1
    args.block_n = int(block_n) if block_n else 0
    args.cta_pair = {None: 0, 128: 1, 256: 2}.get(block_m, 0)  # tile height 128 = one CTA, 256 = a CTA pair
    args.group_m = int(group_size_m) if (block_m is not None or block_n is not None) else 0
    with torch.cuda.device(a.device):
        rc = _lib.lib.tb_gemm_mxfp4(ctypes.byref(args), _lib.current_stream_ptr(a.device))
    _lib.check(rc, "tb_gemm_mxfp4")
    return c


@torch.library.custom_op("tritonblas::_addmm", mutates_args=())
def _addmm(bias: torch.Tensor, a: torch.Tensor, b: torch.Tensor, enable_streamk: Optional[bool] = False,
           sk_grid: Optional[int] = None, work_stealing: Optional[bool] = False) -> torch.Tensor:
    assert a.shape[1] == b.shape[0], "Incompatible A-B Dimensions"
    out = a.new_empty(a.shape[0], b.shape[1])
    selector = _selector_for(a, b, bias.dtype, enable_streamk)
    if enable_streamk:
        streamk_matmul_lt(a, b, out, selector, None, bias=bias, sk_grid=sk_grid, work_stealing=work_stealing)
    else:
        persistent_matmul_lt(a, b, out, selector, None, bias=bias, work_stealing=work_stealing)
    return out


@_addmm.register_fake
def _(bias, a, b, enable_streamk=False, sk_grid=None, work_stealing=False):
    return a.new_empty(a.shape[0], b.shape[1])


def _setup_context_addmm_backwards(ctx, inputs, output):
    bias, a, b, enable_streamk, sk_grid, work_stealing = inputs
    ctx.save_for_backward(a, b)
    ctx.enable_streamk, ctx.sk_grid, ctx.work_stealing = enable_streamk, sk_grid, work_stealing


def _addmm_backwards(ctx, grad_output):
    a, b = ctx.saved_tensors
    kw = dict(enable_streamk=ctx.enable_streamk, sk_grid=ctx.sk_grid, work_stealing=ctx.work_stealing)
    g = grad_output.contiguous()
    grad_bias = grad_output.sum(dim=0) if ctx.needs_input_grad[0] else None
    grad_a = matmul(g, b.T.contiguous(), **kw) if ctx.needs_input_grad[1] else None
    grad_b = matmul(a.T.contiguous(), g, **kw) if ctx.needs_input_grad[2] else None
    return grad_bias, grad_a, grad_b, None, None, None


_addmm.register_autograd(_addmm_backwards, setup_context=_setup_context_addmm_backwards)


@torch.library.custom_op("tritonblas::_addmm_out", mutates_args={"out"})
def _addmm_out(bias: torch.Tensor, a: torch.Tensor, b: torch.Tensor, out: torch.Tensor,
               enable_streamk: Optional[bool] = False, sk_grid: Optional[int] = None,
               work_stealing: Optional[bool] = False) -> None:
    assert a.shape[1] == b.shape[0], "Incompatible A-B Dimensions"
    selector = _selector_for(a, b, bias.dtype, enable_streamk)
    if enable_streamk:
        streamk_matmul_lt(a, b, out, selector, None, bias=bias, sk_grid=sk_grid, work_stealing=work_stealing)
    else:
        persistent_matmul_lt(a, b, out, selector, None, bias=bias, work_stealing=work_stealing)
    return None


def addmm(bias, a, b, out=None, enable_streamk=False, sk_grid=None, work_stealing=False):
    """bias(N,) + A @ B, bias added in fp32 before the output cast."""
    if out is None:
        return _addmm(bias, a, b, enable_streamk, sk_grid, work_stealing)
    if torch.is_grad_enabled() and (bias.requires_grad or a.requires_grad or b.requires_grad or out.requires_grad):
        raise RuntimeError("tritonblas.addmm(): functions with out=... arguments don't support "
                           "automatic differentiation, but one of the arguments requires grad.")
    return _addmm_out(bias, a, b, out, enable_streamk, sk_grid, work_stealing)
