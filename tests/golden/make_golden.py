"""Generates the golden fixtures in this directory by running the REFERENCE's own code on the CPU.

Run once, where the reference tree is available (its location is given in TRITONBLAS_REF):
    TRITONBLAS_REF=<reference checkout> python tests/golden/make_golden.py
Outputs (committed, small):
    decoders.npz        reference mxfp4_to_f32 on all 256 packed bytes, e8m0_to_f32 on all 256 scale bytes
    mxfp4_quant.npz     inputs and the codes/scales the reference Triton quantiser kernel produced for them
    gemm_monolithic.npz inputs and output of the reference monolithic persistent GEMM kernel (fp16, an even and a
                        ragged-K shape; the interpreter mishandles bf16 stores, so bf16 is not recorded)
How: the reference's Triton kernels are executed by Triton's CPU interpreter (TRITON_INTERPRET=1). The quantiser source
is loaded with one expression rewritten in memory (`tl.log2(amax).floor()` -> `tl.floor(tl.log2(amax))`; the
interpreter lacks the method form); nothing from the reference is written into this repository.
"""
import importlib.util
import os
import sys
import tempfile
import types

os.environ["TRITON_INTERPRET"] = "1"
import numpy as np  # noqa: E402
import torch  # noqa: E402

REF = os.environ.get("TRITONBLAS_REF")
if not REF or not os.path.isdir(REF):
    sys.exit("set TRITONBLAS_REF to a checkout of the reference tree")
OUT = os.path.dirname(os.path.abspath(__file__))


def load_reference_utils():
    src = open(os.path.join(REF, "include/tritonblas/utils.py")).read()
    needle = "tl.log2(amax).floor() - 2"
    assert needle in src
    src = src.replace(needle, "tl.floor(tl.log2(amax)) - 2")
    tmp = tempfile.NamedTemporaryFile("w", suffix="_ref_utils.py", delete=False)
    tmp.write(src)
    tmp.close()
    spec = importlib.util.spec_from_file_location("ref_utils", tmp.name)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def quant_inputs():
    g = torch.Generator().manual_seed(1234)
    cases = {}
    cases["randn"] = torch.randn(64, 128, generator=g)
    cases["randn_small"] = torch.randn(32, 64, generator=g) * 1e-3
    cases["randn_large"] = torch.randn(32, 64, generator=g) * 1e4
    x = torch.randn(16, 64, generator=g)
    x[0] = 0.0                      # all-zero blocks
    x[1, :32] = 0.0
    x[2, 5] = 3.0e38                # near fp32 max
    x[3] = x[3] * 1e-38             # denormal range
    x[4, :8] = torch.tensor([0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])   # rounding ties
    x[4, 8:32] = 0.0
    x[5, :32] = 6.0
    x[6, :32] = -6.0
    x[7, :32] = torch.linspace(-7.0, 7.0, 32)
    x[8, :32] = 1.75 * 4            # mantissa exactly at the power-of-two round-up threshold
    x[9, :32] = 1.7499999 * 4
    cases["edges"] = x
    # every e2m1 rounding boundary inside one block whose maximum pins the scale at 1.0
    grid = torch.arange(0, 32, dtype=torch.float32) * 0.1875
    grid[-1] = 6.0
    cases["boundaries"] = torch.stack([grid, -grid, grid.flip(0), grid * 0.5])
    cases["bf16_randn"] = torch.randn(32, 96, generator=g).to(torch.bfloat16).to(torch.float32)
    return cases


def main():
    ref = load_reference_utils()
    # decoders over every byte value
    all_bytes = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(1, 256)
    e2m1 = ref.mxfp4_to_f32(all_bytes.clone()).numpy()
    e8m0 = ref.e8m0_to_f32(all_bytes.clone()).numpy()
    np.savez_compressed(os.path.join(OUT, "decoders.npz"), bytes=all_bytes.numpy(), e2m1=e2m1,
                        e8m0_bits=e8m0.view(np.uint32))
    # quantiser
    out = {}
    for name, x in quant_inputs().items():
        q, s = ref.dynamic_mxfp4_quant(x.contiguous())
        out[name + "_x"] = x.numpy()
        out[name + "_codes"] = q.numpy()
        out[name + "_scales"] = s.numpy()
        print(name, tuple(x.shape), "->", tuple(q.shape), tuple(s.shape))
    np.savez_compressed(os.path.join(OUT, "mxfp4_quant.npz"), **out)
    # monolithic GEMM kernel
    pkg = types.ModuleType("tritonblas")
    pkg.__path__ = [os.path.join(REF, "include/tritonblas")]
    sys.modules["tritonblas"] = pkg
    from tritonblas.kernels.persistent_gemm_monolithic import persistent_matmul as mono
    gem = {}
    for tag, dt, (M, N, K), (BM, BN, BK) in (("f16", torch.float16, (64, 96, 128), (32, 32, 32)),
                                               ("f16_ragged", torch.float16, (48, 80, 72), (16, 16, 32))):
        g = torch.Generator().manual_seed(7)
        a = torch.randn(M, K, generator=g).to(dt)
        b = torch.randn(K, N, generator=g).to(dt)
        c = torch.zeros(M, N, dtype=dt)
        tiles = -(-M // BM) * -(-N // BN)
        mono[(tiles,)](a, b, c, None, None, None, M, N, K, a.stride(0), b.stride(1), c.stride(0), c.stride(1), 0,
                       stride_ak=a.stride(1), stride_bk=b.stride(0), BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK,
                       GROUP_SIZE_M=2, NUM_SMS=tiles, NUM_XCDS=1, CHUNK_SIZE=1, BIAS=False, EVEN_K=(K % BK == 0),
                       CACHE_MODIFIER_A=None, CACHE_MODIFIER_B=None, QUANTIZED=False, ALLOW_TF32=True)
        gem[tag + "_a"] = a.view(torch.int16).numpy()
        gem[tag + "_b"] = b.view(torch.int16).numpy()
        gem[tag + "_c"] = c.view(torch.int16).numpy()
        print("gemm", tag, (M, N, K), "max|c|", c.float().abs().max().item())
    np.savez_compressed(os.path.join(OUT, "gemm_monolithic.npz"), **gem)


if __name__ == "__main__":
    main()
