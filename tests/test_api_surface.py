"""The drop-in boundary on the Python side: the reference's package name, exports and import paths resolve to this
implementation, and its pure-Python known-answer tests keep passing.

Reference: include/tritonblas/__init__.py:1-7 (exports), tests/test_lds_estimation.py:47-114 (shared-memory estimator
known answers), tests/test_matmul_lt.py:5 and tests/test_matmul_fp4.py:10 (import paths), origami.py:349-416 attribute
surface read by callers."""
import inspect

import pytest


def test_reference_package_name_and_exports():
    import tritonblas
    import tritonblas_b200
    for name in ("matmul", "matmul_a8w8", "matmul_lt", "matmul_a8w8_lt", "matmul_fp4", "addmm", "MatmulConfig",
                 "matmul_preamble", "do_bench", "OrigamiMatmulSelector"):
        assert getattr(tritonblas, name) is getattr(tritonblas_b200, name), name
    # import paths the reference's tests and examples use
    from tritonblas.utils import generate_matmul_inputs, dynamic_mxfp4_quant, mxfp4_to_f32, e8m0_to_f32  # noqa: F401
    from tritonblas.origami import estimate_triton_lds_bytes, check_triton_lds_capacity  # noqa: F401
    from tritonblas.config import MatmulConfig, matmul_preamble  # noqa: F401
    from tritonblas.bench import do_bench
    assert do_bench is tritonblas.do_bench


def test_do_bench_signature_matches_reference():
    import tritonblas
    params = inspect.signature(tritonblas.do_bench).parameters
    assert list(params) == ["fn", "reset_fn", "preamble_fn", "n_warmup", "n_repeat", "quantiles", "return_mode"]
    assert params["n_warmup"].default == 25 and params["n_repeat"].default == 100
    assert params["return_mode"].default == "mean" and params["quantiles"].default is None


def test_entry_point_signatures_keep_reference_argument_order():
    import tritonblas
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(tritonblas.matmul)[:5] == ["a", "b", "out", "enable_streamk", "sk_grid"]
    assert sig(tritonblas.matmul_lt)[:6] == ["a", "b", "c", "selector", "config", "enable_streamk"]
    assert sig(tritonblas.matmul_a8w8)[:6] == ["a", "b", "a_scale", "b_scale", "c", "enable_streamk"]
    assert sig(tritonblas.matmul_a8w8_lt)[:8] == ["a", "b", "a_scale", "b_scale", "c", "selector", "config", "enable_streamk"]
    assert sig(tritonblas.matmul_fp4)[:5] == ["a", "b", "c", "a_scales", "b_scales"]
    assert sig(tritonblas.addmm)[:4] == ["bias", "a", "b", "out"]
    assert sig(tritonblas.OrigamiMatmulSelector.__init__)[1:8] == ["m", "n", "k", "a_dtype", "b_dtype", "out_dtype", "device"]
    # extensions beyond the reference are keyword arguments behind the reference's own, off by default
    for f in (tritonblas.matmul_lt, tritonblas.matmul_a8w8_lt):
        p = inspect.signature(f).parameters["static_b"]
        assert p.default is False and list(inspect.signature(f).parameters)[-1] == "static_b"


class TestEstimateTritonLdsBytes:
    """Known answers of the reference's shared-memory estimator (tests/test_lds_estimation.py:47-114)."""

    def test_one_stage_keeps_the_larger_tile(self):
        from tritonblas.origami import estimate_triton_lds_bytes as est
        assert est(128, 128, 64, 2, 2, 1) == 128 * 64 * 2
        assert est(256, 64, 64, 2, 2, 1) == 256 * 64 * 2
        assert est(64, 256, 64, 2, 2, 1) == 64 * 256 * 2

    def test_pipelined_stages_keep_copies_of_both(self):
        from tritonblas.origami import estimate_triton_lds_bytes as est
        assert est(128, 128, 64, 2, 2, 2) == 32768
        assert est(256, 256, 64, 2, 2, 2) == 65536
        assert est(128, 128, 64, 2, 2, 3) == 65536
        assert est(128, 128, 64, 2, 2, 4) == 3 * est(128, 128, 64, 2, 2, 2)
        assert est(128, 64, 64, 2, 2, 2) == 24576
        assert est(256, 128, 64, 2, 2, 2) == 49152
        assert est(64, 64, 32, 2, 2, 2) == 8192
        assert est(128, 256, 64, 2, 2, 2) == 49152

    def test_element_sizes(self):
        from tritonblas.origami import estimate_triton_lds_bytes as est
        assert est(64, 64, 32, 4, 4, 2) == 16384
        assert est(128, 128, 32, 4, 4, 2) == 32768
        assert est(128, 128, 64, 4, 4, 2) == 65536
        assert est(128, 128, 64, 1, 2, 2) == 24576                      # mixed A / B element sizes
        assert est(128, 128, 64, 0.5, 0.5, 2) == est(128, 128, 64, 2, 2, 2) / 4 > 0   # sub-byte types are not free


class TestCheckTritonLdsCapacity:
    """tests/test_lds_estimation.py:117-153 of the reference."""

    def test_capacity(self):
        from tritonblas.origami import check_triton_lds_capacity as fits
        assert fits(64, 64, 32, 2, 2, 65536, 2) is True
        assert fits(256, 256, 64, 4, 4, 65536, 2) is False
        assert fits(256, 256, 64, 2, 2, 65536, 2) is True
        assert fits(128, 128, 64, 2, 2, 65536, 3) is True       # exactly 65536
        assert fits(128, 128, 64, 2, 2, 65536, 4) is False
        assert fits(128, 128, 64, 0.5, 0.5, 0, 2) is False


def test_selector_attribute_surface_without_a_gpu():
    """What reference callers read from a selector (matmul.py:85-89,113,140,234,305; config.py:104-118)."""
    import torch
    import tritonblas
    sel = tritonblas.OrigamiMatmulSelector(4096, 4096, 4096, torch.bfloat16, torch.bfloat16, torch.bfloat16,
                                           torch.device("cuda", 0))
    for attr in ("block_m", "block_n", "block_k", "group_m", "num_sms", "num_stages", "waves_per_eu", "even_k", "sk_grid",
                 "COUNTERS_PER_XCD", "_N_CU", "_ACTIVE_CU"):
        assert getattr(sel, attr) is not None, attr
    assert sel._hardware.N_CU == 148 and sel._hardware.NUM_XCD == 1 and sel.num_sms == 1
    local, glob = sel.hierarchical_split(1)
    assert local >= 1 and glob >= 0
    with pytest.raises(ValueError):
        tritonblas.OrigamiMatmulSelector(64, 64, 64, torch.int64, torch.int64, torch.int64, torch.device("cuda", 0))
