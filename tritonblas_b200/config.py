"""Caller-owned workspace for GEMM launches; same surface as the reference's ``MatmulConfig`` /
``matmul_preamble`` (include/tritonblas/config.py:10-134).

The stream-K workspace is one byte buffer: 4 KB of per-program flags followed by one fp32 partial tile per CTA.
``locks`` and ``P`` are views into it with the reference's shapes. Flags carry a per-launch epoch instead of 0/1, so
nothing has to be cleared between launches; ``reset()`` still exists and is safe to call.
"""
import ctypes

import torch

from . import _lib

COUNTER_STRIDE = 64  # int32 elements between counters: 256 bytes, one per L2 line pair (config.py:3-5)
MAX_SK_TILES = 512
_FLAG_BYTES = 4096


class MatmulConfig:
    def __init__(self, device, workspace, sk_grid, block_size, tile_counter, global_counter, mask):
        self.device = device
        self.workspace = workspace
        self.epoch = 0
        self.locks = workspace[:sk_grid]
        self.P = workspace[_FLAG_BYTES:_FLAG_BYTES + sk_grid * block_size * 4].view(torch.float32).view(sk_grid, block_size)
        self.tile_counter = tile_counter
        self.streamk_tile_counter = tile_counter.clone()
        self.global_counter = global_counter
        self.global_atomic = False
        self.mask = mask
        self.sk_iter_counter = torch.zeros(COUNTER_STRIDE, device=device, dtype=torch.int32)
        self.sk_locks = self.sk_done = self.sk_P = None
        # Launches made with this config: bound of every device-side wait in milliseconds (0 = the library's 2 s) and the
        # library's measurement / test switches (tb_gemm_args.debug_flags; 0 in production).
        self.wait_timeout_ms = 0
        self.debug_flags = 0

    def next_epoch(self):
        self.epoch = (self.epoch % 0xFFFFFFF0) + 1
        if self.epoch == 1 and self.workspace is not None:
            self.workspace[:_FLAG_BYTES].zero_()
        return self.epoch

    def reset(self, streamk=False, work_stealing=False):
        """Clear mutable launch state (config.py:54-75). Enqueued on the current stream."""
        if work_stealing:
            self.tile_counter.zero_()
            self.global_counter.zero_()
        if streamk:
            self.workspace[:_FLAG_BYTES].zero_()
            self.epoch = 0
            self.sk_iter_counter.zero_()

    def __repr__(self):
        return (f"MatmulConfig(device={self.device!r}, tile_counter={list(self.tile_counter.shape)}, "
                f"locks={list(self.locks.shape)}, P={list(self.P.shape)})")


def workspace_bytes(cfg, sk_grid=0):
    return int(_lib.lib.tb_gemm_workspace_bytes(ctypes.byref(cfg), int(sk_grid)))


def matmul_preamble(selector, device=None):
    """Allocate the buffers GEMM launches with ``selector`` may need (config.py:86-134)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    cfg = selector._cfg
    sk_grid = max(selector.sk_grid, 1)
    nbytes = workspace_bytes(cfg, sk_grid)
    workspace = torch.zeros(nbytes, device=device, dtype=torch.uint8)
    counters = selector._hardware.NUM_XCD * selector.COUNTERS_PER_XCD
    tile_counter = torch.zeros(counters * COUNTER_STRIDE, device=device, dtype=torch.int32)
    global_counter = torch.zeros(COUNTER_STRIDE, device=device, dtype=torch.int32)
    mask = torch.ones(selector._N_CU, dtype=torch.int32, device=device)
    if selector._ACTIVE_CU < selector._N_CU:
        mask[selector._ACTIVE_CU:] = 0
    return MatmulConfig(device, workspace, sk_grid, selector.block_m * selector.block_n, tile_counter, global_counter, mask)
