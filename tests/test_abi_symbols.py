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


def test_ctypes_structures_mirror_the_header_field_for_field(tmp_path):
    """Every structure of the C header, compiled by the host C compiler, has the size the ctypes mirror has, and every
    field sits at the same offset: a field added on one side only cannot go unnoticed."""
    import os
    import re
    import shutil
    import subprocess
    from tritonblas_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no host C compiler")
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    header = os.path.join(here, "include", "tritonblas_b200.h")
    text = open(header).read()
    pairs = {"tb_problem": _lib.Problem, "tb_config": _lib.Config, "tb_gemm_args": _lib.GemmArgs, "tb_mxfp4_args": _lib.Mxfp4Args}
    lines = ["#include <stdio.h>", "#include <stddef.h>", f'#include "{header}"', "int main(void) {"]
    for cname, mirror in pairs.items():
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), text, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for stmt in body.split(";"):
            for piece in stmt.split(","):       # "int32_t m, n, k" declares three fields
                found = re.findall(r"(\w+)\s*(?:\[\d+\])?\s*$", piece.strip())
                names += found
        assert names == [f[0] for f in mirror._fields_], (cname, names, [f[0] for f in mirror._fields_])
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for n in names:
            lines.append(f'printf("{cname}.{n} %zu\\n", offsetof({cname}, {n}));')
    lines += ["return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-std=c11", "-o", str(exe), str(src)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, mirror in pairs.items():
        assert int(out[cname]) == ctypes.sizeof(mirror), cname
        for fname, _ in mirror._fields_:
            assert int(out[f"{cname}.{fname}"]) == getattr(mirror, fname).offset, (cname, fname)


def test_integration_stub_lists_the_same_fields_as_the_header():
    """The reference-side ctypes stub shown in the integration guide names every field of tb_gemm_args and tb_config, in
    order."""
    from tritonblas_b200 import _lib
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    args_block = text[text.index("class _Args(ctypes.Structure)"):]
    args_block = args_block[:args_block.index("_DT = ")]
    names = re.findall(r'\("(\w+)",\s*ctypes\.', args_block)
    assert names == [f[0] for f in _lib.GemmArgs._fields_], names
    cfg_block = text[text.index("class _Cfg(ctypes.Structure)"):text.index("class _Args(ctypes.Structure)")]
    cfg_names = re.findall(r'"(\w+)"', cfg_block)
    assert cfg_names == [f[0] for f in _lib.Config._fields_], cfg_names
