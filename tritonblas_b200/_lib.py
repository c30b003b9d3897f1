"""ctypes binding of libtritonblas_b200.so (the C ABI declared in include/tritonblas_b200.h).

There is no fallback: if the shared library has not been built, importing the package raises with the build command.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtritonblas_b200.so")

# element type codes (TB_DTYPE_* in the header)
F16, BF16, F32, E4M3, E5M2, U8, F4, I8 = range(8)

DTYPE_CODE = {
    torch.float16: F16,
    torch.bfloat16: BF16,
    torch.float32: F32,
    torch.float8_e4m3fn: E4M3,
    torch.float8_e5m2: E5M2,
    torch.uint8: U8,
    torch.int8: I8,
}


class Problem(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "m", "n", "k", "a_dtype", "b_dtype", "c_dtype", "a_mn_major", "b_mn_major", "streamk", "mx_block_size",
        "num_sms", "device", "max_halves")]


class Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in (
        "block_m", "block_n", "block_k", "group_m", "stages", "cta_pair", "grid", "sk_grid", "num_sms", "smem_bytes",
        "tmem_cols")] + [("predicted_us", ctypes.c_float), ("predicted_sk_us", ctypes.c_float), ("n_halves", ctypes.c_int32),
                                ("swap_ab", ctypes.c_int32)]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
        ("a_dtype", ctypes.c_int32), ("b_dtype", ctypes.c_int32), ("c_dtype", ctypes.c_int32),
        ("a", ctypes.c_void_p), ("a_stride_m", ctypes.c_int64), ("a_stride_k", ctypes.c_int64),
        ("b", ctypes.c_void_p), ("b_stride_k", ctypes.c_int64), ("b_stride_n", ctypes.c_int64),
        ("c", ctypes.c_void_p), ("c_stride_m", ctypes.c_int64), ("c_stride_n", ctypes.c_int64),
        ("a_scale", ctypes.c_void_p), ("b_scale", ctypes.c_void_p),
        ("bias", ctypes.c_void_p), ("bias_stride", ctypes.c_int64), ("bias_dtype", ctypes.c_int32),
        ("allow_tf32", ctypes.c_int32), ("streamk", ctypes.c_int32), ("sk_grid", ctypes.c_int32),
        ("workspace", ctypes.c_void_p), ("workspace_bytes", ctypes.c_int64), ("epoch", ctypes.c_uint32),
        ("group_offsets", ctypes.c_void_p), ("num_groups", ctypes.c_int32),
        ("c_copies", ctypes.POINTER(ctypes.c_void_p)), ("num_c_copies", ctypes.c_int32),
        ("tile_counter", ctypes.c_void_p), ("epilogue_op", ctypes.c_int32),
        ("wait_timeout_ms", ctypes.c_int32), ("debug_flags", ctypes.c_int32),
        ("a_gather_index", ctypes.c_void_p), ("a_rows", ctypes.c_int64), ("c_copies_tile_limit", ctypes.c_int32), ("static_operands", ctypes.c_int32),
    ]


class Mxfp4Args(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int32), ("n", ctypes.c_int32), ("k", ctypes.c_int32),
        ("a", ctypes.c_void_p), ("a_row_stride", ctypes.c_int64),
        ("b", ctypes.c_void_p), ("b_row_stride", ctypes.c_int64),
        ("c", ctypes.c_void_p), ("c_stride_m", ctypes.c_int64), ("c_stride_n", ctypes.c_int64), ("c_dtype", ctypes.c_int32),
        ("a_scales", ctypes.c_void_p), ("b_scales", ctypes.c_void_p), ("scales_in_atoms", ctypes.c_int32),
        ("block_n", ctypes.c_int32), ("cta_pair", ctypes.c_int32), ("group_m", ctypes.c_int32),
    ]


def _load():
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python tritonblas_b200/csrc/build.py` "
            "(nvcc, sm_100a). tritonblas_b200 has no CPU or PyTorch fallback path.")
    lib = ctypes.CDLL(LIB_PATH)
    lib.tb_select.argtypes = [ctypes.POINTER(Problem), ctypes.POINTER(Config)]
    lib.tb_select.restype = ctypes.c_int
    lib.tb_gemm_workspace_bytes.argtypes = [ctypes.POINTER(Config), ctypes.c_int32]
    lib.tb_gemm_workspace_bytes.restype = ctypes.c_int64
    lib.tb_gemm.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(Config), ctypes.c_void_p]
    lib.tb_gemm.restype = ctypes.c_int
    lib.tb_gemm_tile_count.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(Config)]
    lib.tb_gemm_tile_count.restype = ctypes.c_int
    lib.tb_push_c_tiles.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(Config), ctypes.c_int32, ctypes.c_void_p]
    lib.tb_push_c_tiles.restype = ctypes.c_int
    lib.tb_gemm_streamk_builtin.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(Config), ctypes.c_void_p,
                                            ctypes.POINTER(ctypes.c_int32)]
    lib.tb_gemm_streamk_builtin.restype = ctypes.c_int
    lib.tb_grouped_gemm.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(Config), ctypes.c_void_p]
    lib.tb_grouped_gemm.restype = ctypes.c_int
    lib.tb_swiglu.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                              ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.tb_swiglu.restype = ctypes.c_int
    lib.tb_moe_combine.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                   ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                   ctypes.c_void_p]
    lib.tb_moe_combine.restype = ctypes.c_int
    lib.tb_moe_gather_rows.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                       ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p]
    lib.tb_moe_gather_rows.restype = ctypes.c_int
    lib.tb_moe_dispatch_peers.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int64, ctypes.c_int64,
                                          ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                          ctypes.c_void_p]
    lib.tb_moe_dispatch_peers.restype = ctypes.c_int
    lib.tb_moe_count.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p,
                                 ctypes.c_void_p, ctypes.c_void_p]
    lib.tb_moe_count.restype = ctypes.c_int
    lib.tb_moe_plan.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int32,
                                ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_void_p]
    lib.tb_moe_plan.restype = ctypes.c_int
    lib.tb_moe_combine_peers.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p,
                                         ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                         ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p]
    lib.tb_moe_combine_peers.restype = ctypes.c_int
    lib.tb_tma_stream_probe.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.tb_tma_stream_probe.restype = ctypes.c_int32
    lib.tb_peer_store_probe.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_int64, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.tb_peer_store_probe.restype = ctypes.c_int
    lib.tb_gemm_mxfp4.argtypes = [ctypes.POINTER(Mxfp4Args), ctypes.c_void_p]
    lib.tb_gemm_mxfp4.restype = ctypes.c_int
    lib.tb_mxfp4_quant.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                   ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32,
                                   ctypes.c_void_p]
    lib.tb_mxfp4_quant.restype = ctypes.c_int
    lib.tb_mxfp4_quant_atoms.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                         ctypes.c_int32, ctypes.c_void_p]
    lib.tb_mxfp4_quant_atoms.restype = ctypes.c_int
    lib.tb_mxfp4_atoms_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    lib.tb_mxfp4_atoms_bytes.restype = ctypes.c_int64
    lib.tb_mxfp4_scales_to_atoms.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                             ctypes.c_void_p, ctypes.c_void_p]
    lib.tb_mxfp4_scales_to_atoms.restype = ctypes.c_int
    lib.tb_fp8_quant_rows.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                      ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    lib.tb_fp8_quant_rows.restype = ctypes.c_int
    lib.tb_device_status.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32)]
    lib.tb_device_status.restype = ctypes.c_int
    lib.tb_device_info.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32)]
    lib.tb_device_info.restype = ctypes.c_int
    lib.tb_status_string.argtypes = [ctypes.c_int]
    lib.tb_status_string.restype = ctypes.c_char_p
    lib.tb_last_cuda_error.argtypes = []
    lib.tb_last_cuda_error.restype = ctypes.c_char_p
    lib.tb_launch_count.argtypes = []
    lib.tb_launch_count.restype = ctypes.c_int64
    return lib


lib = _load()


class TritonBlasError(RuntimeError):
    """A C-ABI call returned a non-zero status."""


def check(rc, what="tritonblas_b200"):
    if rc != 0:
        msg = lib.tb_status_string(rc).decode()
        if rc == 5:
            msg += f" ({lib.tb_last_cuda_error().decode()})"
        raise TritonBlasError(f"{what}: {msg} [code {rc}]")


def device_status(device=None):
    """Synchronise `device` and return (then clear) the failure code kernels record when a bounded wait gives up."""
    if device is None:
        device = torch.cuda.current_device()
    out = ctypes.c_int32(0)
    check(lib.tb_device_status(int(device), ctypes.byref(out)), "tb_device_status")
    return out.value


_failure_hooks = []  # callables run when a device-side failure is reported (e.g. to zero shared launch state)


def raise_on_device_failure(device=None):
    code = device_status(device)
    if code != 0:
        for hook in _failure_hooks:
            hook()
        raise TritonBlasError(f"device-side failure: {lib.tb_status_string(code).decode()} [code {code}]")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream_ptr(device=None):
    """The current CUDA stream of `device` as a pointer (the raw-handle getter when torch has it: it skips building a
    torch.cuda.Stream object on every launch)."""
    if _raw_stream is not None:
        if device is None:
            index = torch.cuda.current_device()
        elif isinstance(device, int):
            index = device
        else:
            index = device.index if device.index is not None else torch.cuda.current_device()
        return ctypes.c_void_p(_raw_stream(index))
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
