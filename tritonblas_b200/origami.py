"""Tile / schedule selector with the attribute surface of the reference's ``OrigamiMatmulSelector``
(include/tritonblas/origami.py:62-347). The analytical model lives in the C-ABI library (``tb_select``), as the
reference's lives in its native ``origami`` extension; this class only marshals the problem and exposes the result.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def estimate_triton_lds_bytes(block_m, block_n, block_k, bytes_a, bytes_b, num_stages=2):
    """Shared-memory bytes of a software-pipelined A/B tile pair, as the reference estimates them
    (include/tritonblas/origami.py:9-44): one stage keeps the larger tile, n stages keep n-1 copies of both."""
    tile_a = block_m * block_k * bytes_a
    tile_b = block_k * block_n * bytes_b
    if num_stages <= 1:
        return max(tile_a, tile_b)
    return (num_stages - 1) * (tile_a + tile_b)


def check_triton_lds_capacity(block_m, block_n, block_k, bytes_a, bytes_b, lds_capacity, num_stages=2):
    """True when :func:`estimate_triton_lds_bytes` fits ``lds_capacity`` (include/tritonblas/origami.py:47-59)."""
    return estimate_triton_lds_bytes(block_m, block_n, block_k, bytes_a, bytes_b, num_stages) <= lds_capacity


class _Hardware:
    """What callers read from ``selector._hardware``: B200 has one L2 domain, so one "XCD"."""

    def __init__(self, n_cu, smem):
        self.N_CU = n_cu
        self.NUM_XCD = 1
        self.CU_per_L2 = n_cu
        self.lds_capacity = smem


_STR_DTYPES = {"f16": _lib.F16, "bf16": _lib.BF16, "f32": _lib.F32, "f8": _lib.E4M3, "f4": _lib.F4, "i8": _lib.I8}


def _dtype_code(dt):
    if isinstance(dt, str):
        if dt in _STR_DTYPES:
            return _STR_DTYPES[dt]
    elif dt in _lib.DTYPE_CODE:
        return _lib.DTYPE_CODE[dt]
    raise ValueError(f"Unsupported data type for the B200 GEMM selector: {dt}")


class OrigamiMatmulSelector:
    """Chooses tile, CTA pairing, stage count and grids for one GEMM problem on B200.

    Positional arguments and properties match the reference class; ``a_mn_major`` / ``b_mn_major`` are additions
    (the reference assumes the T,N layout, origami.py:479-480) that tell the model which operand is stored with its
    M or N axis contiguous.
    """

    COUNTERS_PER_XCD = 4

    @staticmethod
    def estimate_triton_lds(block_m, block_n, block_k, bytes_a, bytes_b, num_stages=2):
        return estimate_triton_lds_bytes(block_m, block_n, block_k, bytes_a, bytes_b, num_stages)

    def __init__(self, m, n, k, a_dtype, b_dtype, out_dtype, device=None, mx_block_size=0, streamk=False,
                 total_cus=None, active_cus=None, num_stages=2, a_mn_major=False, b_mn_major=False, max_halves=0):
        self._m, self._n, self._k = int(m), int(n), int(k)
        self._max_halves = int(max_halves)  # 1: narrow tiles only (grouped launches)
        self.streamk = bool(streamk)
        self._num_stages = num_stages
        self._mx_block_size = mx_block_size
        self._a_code = _dtype_code(a_dtype)
        self._b_code = _dtype_code(b_dtype)
        self._c_code = _dtype_code(out_dtype)
        if isinstance(device, torch.device):
            dev_index = device.index if device.index is not None else (
                torch.cuda.current_device() if torch.cuda.is_available() else 0)
        elif device is None:
            dev_index = torch.cuda.current_device() if torch.cuda.is_available() else 0
        else:
            dev_index = int(device)
        self._device_index = dev_index
        n_sms, smem = ctypes.c_int32(0), ctypes.c_int32(0)
        if _lib.lib.tb_device_info(dev_index, ctypes.byref(n_sms), ctypes.byref(smem)) != 0:
            n_sms, smem = ctypes.c_int32(148), ctypes.c_int32(232448)  # B200 constants when no device is visible
        self._N_CU = int(total_cus) if total_cus is not None else n_sms.value
        self._ACTIVE_CU = int(active_cus) if active_cus is not None else self._N_CU
        self._hardware = _Hardware(self._N_CU, smem.value)
        self._configs = {}
        self._layout = (bool(a_mn_major), bool(b_mn_major))
        self._cfg = self.config_for(*self._layout)
        tiles_m = -(-self._m // self._cfg.block_m)
        tiles = tiles_m * -(-self._n // self._cfg.block_n)
        # work-stealing bookkeeping kept for callers that size counter buffers from it (origami.py:266-286)
        self.COUNTERS_PER_XCD = 8 if tiles <= 512 else 4 if tiles <= 1536 else 2 if tiles <= 2048 else 1

    def config_for(self, a_mn_major, b_mn_major):
        """Configuration for a given operand layout (cached); the default layout is the constructor's."""
        key = (bool(a_mn_major), bool(b_mn_major))
        if key not in self._configs:
            p = _lib.Problem(m=self._m, n=self._n, k=self._k, a_dtype=self._a_code, b_dtype=self._b_code,
                             c_dtype=self._c_code, a_mn_major=int(key[0]), b_mn_major=int(key[1]),
                             streamk=int(self.streamk), mx_block_size=int(self._mx_block_size or 0),
                             num_sms=min(self._ACTIVE_CU, self._N_CU), device=self._device_index,
                             max_halves=self._max_halves)
            cfg = _lib.Config()
            rc = _lib.lib.tb_select(ctypes.byref(p), ctypes.byref(cfg))
            if rc != 0:
                raise ValueError(f"No valid B200 GEMM configuration for m={self._m} n={self._n} k={self._k}: "
                                 f"{_lib.lib.tb_status_string(rc).decode()}")
            self._configs[key] = cfg
        return self._configs[key]

    def override(self, **fields):
        """Force fields of the launch configuration (block_n, n_halves, cta_pair, stages, group_m, grid, sk_grid) for every
        layout; block_m follows cta_pair. For tuning sweeps and tests; the library re-validates the result."""
        for key in [(False, False), (False, True), (True, False), (True, True)]:
            cfg = self.config_for(*key)
            for name, value in fields.items():
                if not hasattr(cfg, name):
                    raise AttributeError(name)
                setattr(cfg, name, int(value))
            cfg.block_m = 128 * (2 if cfg.cta_pair == 2 else 1)
            if "cta_pair" in fields or "block_n" in fields or "n_halves" in fields:
                # grids, ring depth and tile order follow the tile shape unless they are forced as well
                pair = 2 if cfg.cta_pair == 2 else 1
                halves = max(cfg.n_halves, 1)
                programs = max(cfg.num_sms // pair, 1)
                tiles_m = -(-self._m // cfg.block_m)
                tiles = tiles_m * -(-self._n // (cfg.block_n * halves))
                if "grid" not in fields:
                    cfg.grid = min(programs, tiles)
                if "sk_grid" not in fields:
                    cfg.sk_grid = min(programs, tiles * -(-self._k // cfg.block_k))
                if "stages" not in fields and not self._mx_block_size:
                    stage = (128 * 128 + halves * (cfg.block_n // pair) * 128 + 1023) & ~1023
                    cfg.stages = max(2, min(12, (self._hardware.lds_capacity - 2048 - 16384) // stage))
                    if cfg.swap_ab:     # same cap as the selector's: about 160 KB requested ahead per SM
                        cfg.stages = min(cfg.stages, max(4, 168 * 1024 // stage))
                if "group_m" not in fields:
                    g = round((programs * cfg.block_n * halves / cfg.block_m) ** 0.5)
                    cfg.group_m = max(1, min(tiles_m, g))
        return self

    def hierarchical_split(self, num_xcds):
        """(local tiles per domain, global tiles) split of the tile space, same rule as origami.py:288-311."""
        tiles = -(-self._m // self.block_m) * -(-self._n // self.block_n)
        per_cu = tiles / max(self._hardware.NUM_XCD * self._hardware.CU_per_L2, 1)
        local_frac = max(0.5, 1.0 - max(0.0, per_cu - 4.0) * 0.05)
        local = max(int(tiles * local_frac) // num_xcds, 1)
        return local, tiles - local * num_xcds

    block_m = property(lambda self: self._cfg.block_m)
    block_n = property(lambda self: self._cfg.block_n)
    block_k = property(lambda self: self._cfg.block_k)
    group_m = property(lambda self: self._cfg.group_m)
    num_sms = property(lambda self: self._hardware.NUM_XCD)  # the reference's name for its XCD count
    num_stages = property(lambda self: self._cfg.stages)
    waves_per_eu = property(lambda self: 1)
    even_k = property(lambda self: self._k % self.block_k == 0)
    sk_grid = property(lambda self: self._cfg.sk_grid)
    grid = property(lambda self: self._cfg.grid)
    cta_pair = property(lambda self: self._cfg.cta_pair)
    predicted_us = property(lambda self: self._cfg.predicted_sk_us if self.streamk else self._cfg.predicted_us)

    def __repr__(self):
        c = self._cfg
        return (f"OrigamiMatmulSelector(m={self._m}, n={self._n}, k={self._k}, tile={c.block_m}x{c.block_n}x{c.block_k}, "
                f"cta_pair={c.cta_pair}, stages={c.stages}, group_m={c.group_m}, grid={c.grid}, sk_grid={c.sk_grid})")
