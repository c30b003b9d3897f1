"""The shared library loads on a machine without a GPU and exports every entry point the public header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(tb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported():
    from tritonblas_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared()
    assert len(declared) >= 8
    missing = [n for n in declared if not hasattr(lib, n)]
    assert not missing, missing


def test_status_strings():
    from tritonblas_b200 import _lib
    assert _lib.lib.tb_status_string(0) == b"ok"
    assert b"stream-K" in _lib.lib.tb_status_string(4)
    assert b"device" in _lib.lib.tb_status_string(105)


def test_struct_sizes_match_header_layout():
    from tritonblas_b200 import _lib
    assert ctypes.sizeof(_lib.Problem) == 13 * 4
    assert ctypes.sizeof(_lib.Config) == 15 * 4


def test_library_sources_name_no_device_allocator():
    """The library never allocates device memory (its status word and the built-in stream-K scratch are part of the
    library image): no source file calls an allocating or freeing CUDA routine."""
    import glob
    import os
    import re
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pat = re.compile(r"\b(cudaMalloc\w*|cudaFree\w*|cuMemAlloc\w*|cuMemFree\w*|cudaHostAlloc|cuMemCreate)\s*\(")
    for path in glob.glob(os.path.join(here, "tritonblas_b200", "csrc", "*")):
        if path.endswith((".cu", ".cuh", ".cpp", ".h")):
            with open(path) as f:
                assert not pat.search(f.read()), path
