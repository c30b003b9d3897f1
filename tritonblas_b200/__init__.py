"""tritonblas_b200: the tritonBLAS GEMM API on B200, backed by hand-written sm_100a kernels behind a C ABI."""
from .matmul import (matmul, matmul_lt, matmul_a8w8, matmul_a8w8_lt, matmul_fp4, grouped_matmul, addmm, persistent_matmul_lt,
                     streamk_matmul_lt)
from .config import MatmulConfig, matmul_preamble
from .origami import OrigamiMatmulSelector
from .bench import do_bench
from ._lib import TritonBlasError, device_status, raise_on_device_failure

__all__ = ["matmul", "matmul_lt", "matmul_a8w8", "matmul_a8w8_lt", "matmul_fp4", "grouped_matmul", "addmm", "MatmulConfig", "matmul_preamble",
           "OrigamiMatmulSelector", "do_bench", "TritonBlasError", "device_status", "raise_on_device_failure"]
