// Per-row symmetric FP8 (e4m3) quantiser: scale[r] = max(amax(x[r, :]), 1e-8) / 448, q = cast(x * (1 / scale)).
// Same arithmetic, in the same order, as the reference fixture quantize_tensor_per_channel(axis=1)
// (include/tritonblas/utils.py:340-377): fp32 amax, fp32 divide, fp32 reciprocal, fp32 multiply, round-to-nearest-even
// cast. Rows of activations are tokens; rows of a weight stored (N, K) are output channels, so one kernel serves both
// operands of the a8w8 GEMM. One CTA per row: pass 1 reduces the maximum, pass 2 re-reads the row (L1/L2 resident) and
// converts. HBM traffic: 2 bytes in + 1 byte out per element.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common_host.h"

namespace tb {
namespace {

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(u[j] << 16);
    v[2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
  }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[j]));
    v[2 * j] = f.x;
    v[2 * j + 1] = f.y;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) quant_fp8_rows_kernel(const T* __restrict__ x, long long x_stride,
                                                               unsigned char* __restrict__ q, long long q_stride,
                                                               float* __restrict__ scales, int rows, int k) {
  __shared__ float warp_max[8];
  __shared__ float inv_shared;
  const int vecs = k / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + row * x_stride;
    float amax = 0.f;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float f[8];
      load8<T>(xr + v * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = warp_max[0];
      for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
      // torch divides a CUDA tensor by a host scalar as a multiplication by the scalar's fp32 reciprocal; the fixture's
      // `max_abs / dtype_max` therefore rounds this way, and so does this kernel
      const float scale = __fmul_rn(fmaxf(m, 1e-8f), __fdiv_rn(1.0f, 448.0f));
      scales[row] = scale;
      inv_shared = __fdiv_rn(1.0f, scale);
    }
    __syncthreads();
    const float inv = inv_shared;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float f[8];
      load8<T>(xr + v * 8, f);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        lo |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(f[j], inv), __NV_SATFINITE, __NV_E4M3)) << (8 * j);
        hi |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(__fmul_rn(f[4 + j], inv), __NV_SATFINITE, __NV_E4M3)) << (8 * j);
      }
      *reinterpret_cast<uint2*>(q + row * q_stride + v * 8) = make_uint2(lo, hi);
    }
    __syncthreads();
  }
}

}  // namespace
}  // namespace tb

extern "C" int tb_fp8_quant_rows(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* q,
                                 int64_t q_row_stride, float* scales, void* stream) {
  if (x == nullptr || q == nullptr || scales == nullptr || rows < 0 || k < 0 || (k % 8) != 0) return TB_ERR_INVALID;
  if (rows == 0 || k == 0) return TB_OK;
  if (rows > 0x7FFFFFFF || k > 0x7FFFFFFF) return TB_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((x_row_stride * 2) & 15) != 0) return TB_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(q) & 7) != 0 || (q_row_stride & 7) != 0) return TB_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = static_cast<int>(rows < 148 * 16 ? rows : 148 * 16);
  if (x_dtype == TB_DTYPE_BF16)
    tb::quant_fp8_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), x_row_stride,
                                                                  static_cast<unsigned char*>(q), q_row_stride, scales,
                                                                  static_cast<int>(rows), static_cast<int>(k));
  else if (x_dtype == TB_DTYPE_F16)
    tb::quant_fp8_rows_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(x), x_row_stride,
                                                           static_cast<unsigned char*>(q), q_row_stride, scales,
                                                           static_cast<int>(rows), static_cast<int>(k));
  else
    return TB_ERR_UNSUPPORTED;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "quant_fp8_rows_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}
