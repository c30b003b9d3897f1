"""The reference's package name: ``import tritonblas`` resolves to the B200 implementation (``tritonblas_b200``), so code
written against the reference (include/tritonblas/__init__.py:1-7, examples/example_matmul.py:3,14) runs unchanged.

The submodules callers import by path (``tritonblas.utils``, ``tritonblas.origami``, ``tritonblas.config``,
``tritonblas.matmul``, ``tritonblas.bench``) are the implementation's modules under their reference names.
"""
import importlib as _importlib
import sys as _sys

import tritonblas_b200 as _impl
from tritonblas_b200 import *  # noqa: F401,F403
from tritonblas_b200 import __all__ as _impl_all

for _name in ("matmul", "config", "origami", "utils", "bench"):
    _sys.modules[__name__ + "." + _name] = _importlib.import_module("tritonblas_b200." + _name)

# As in the reference, the functions shadow the submodules of the same name on the package object
# (``tritonblas.matmul`` is the function; ``import tritonblas.matmul as mod`` still reaches the module).
from tritonblas_b200.matmul import matmul, matmul_a8w8, matmul_lt, matmul_a8w8_lt, matmul_fp4, addmm  # noqa: E402,F401
from tritonblas_b200.config import MatmulConfig, matmul_preamble  # noqa: E402,F401
from tritonblas_b200.bench import do_bench  # noqa: E402,F401
from tritonblas_b200.origami import OrigamiMatmulSelector  # noqa: E402,F401

__all__ = list(_impl_all)
