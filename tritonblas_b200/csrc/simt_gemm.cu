// CUDA-core GEMM for the cases the tensor-core path does not take:
//   - fp32 operands when tf32 products are not allowed (exact fp32 multiply-add, the reference's
//     ALLOW_TF32=False mode, include/tritonblas/matmul.py:147);
//   - operands whose base pointer or row pitch is not 16-byte aligned, which TMA cannot address
//     (e.g. the reference's K = 970132 bf16 case, tests/test_matmul_lt.py:14).
// 128 x 128 output tile per CTA, 16-deep K slices through shared memory, 8 x 8 accumulators per thread, fp32 accumulate.
// Epilogue order as everywhere: scale -> bias -> cast -> masked store.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <type_traits>

#include "common_host.h"

namespace tb {

namespace {

constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8;

struct SimtParams {
  int M, N, K;
  const void* A; long long a_sm, a_sk; int a_dtype;
  const void* B; long long b_sk, b_sn; int b_dtype;
  void* C; long long c_sm, c_sn; int c_dtype;
  void* c_extra[7]; int num_c_extra;  // further destinations laid out like C (the tensor-core path's fan-out)
  const float* a_scale; const float* b_scale;
  const void* bias; long long bias_stride; int bias_dtype;
};

__device__ __forceinline__ float ld_elem(const void* p, long long i, int dtype) {
  switch (dtype) {
    case TB_DTYPE_F16: return __half2float(reinterpret_cast<const __half*>(p)[i]);
    case TB_DTYPE_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    case TB_DTYPE_F32: return reinterpret_cast<const float*>(p)[i];
    case TB_DTYPE_E4M3: {
      __half_raw h = __nv_cvt_fp8_to_halfraw(reinterpret_cast<const unsigned char*>(p)[i], __NV_E4M3);
      return __half2float(*reinterpret_cast<__half*>(&h));
    }
    case TB_DTYPE_E5M2: {
      __half_raw h = __nv_cvt_fp8_to_halfraw(reinterpret_cast<const unsigned char*>(p)[i], __NV_E5M2);
      return __half2float(*reinterpret_cast<__half*>(&h));
    }
    case TB_DTYPE_I8: return static_cast<float>(reinterpret_cast<const signed char*>(p)[i]);
    default: return 0.f;
  }
}

__device__ __forceinline__ void st_elem(void* p, long long i, int dtype, float v) {
  switch (dtype) {
    case TB_DTYPE_F16: reinterpret_cast<__half*>(p)[i] = __float2half_rn(v); break;
    case TB_DTYPE_BF16: reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
    case TB_DTYPE_F32: reinterpret_cast<float*>(p)[i] = v; break;
    case TB_DTYPE_E4M3:
      reinterpret_cast<unsigned char*>(p)[i] = static_cast<unsigned char>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
      break;
    case TB_DTYPE_I8:
      reinterpret_cast<signed char*>(p)[i] = static_cast<signed char>(__float2int_rn(fminf(fmaxf(v, -128.0f), 127.0f)));
      break;
    default: break;
  }
}

// Acc = float, or int for 8-bit integer operands (exact int32 sums, as the tensor-core integer kind produces).
template <typename Acc>
__global__ void __launch_bounds__(256) simt_gemm_kernel(const SimtParams p) {
  __shared__ Acc As[BK][BM + 4];
  __shared__ Acc Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  Acc acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = Acc(0);

  // Loader mapping follows the contiguous axis of each operand so global reads coalesce for either layout.
  const bool a_kc = (p.a_sk == 1);
  const bool b_nc = (p.b_sn == 1);
  for (int k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; ++i) {
      const int idx = tid + i * 256;
      const int kk = a_kc ? idx % BK : idx / BM;
      const int mm = a_kc ? idx / BK : idx % BM;
      const int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < p.M && gk < p.K) ? static_cast<Acc>(ld_elem(p.A, gm * p.a_sm + gk * p.a_sk, p.a_dtype)) : Acc(0);
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / 256; ++i) {
      const int idx = tid + i * 256;
      const int kk = b_nc ? idx / BN : idx % BK;
      const int nn = b_nc ? idx % BN : idx / BK;
      const int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < p.N && gk < p.K) ? static_cast<Acc>(ld_elem(p.B, gk * p.b_sk + gn * p.b_sn, p.b_dtype)) : Acc(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      Acc a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          if constexpr (std::is_same<Acc, float>::value) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          else acc[i][j] += a[i] * b[j];
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= p.M) continue;
    const float as = p.a_scale ? p.a_scale[gm] : 1.f;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= p.N) continue;
      float v = static_cast<float>(acc[i][j]);
      if (p.a_scale) v *= as;
      if (p.b_scale) v *= p.b_scale[gn];
      if (p.bias) v += ld_elem(p.bias, gn * p.bias_stride, p.bias_dtype);
      st_elem(p.C, gm * p.c_sm + gn * p.c_sn, p.c_dtype, v);
      for (int x = 0; x < p.num_c_extra; ++x) st_elem(p.c_extra[x], gm * p.c_sm + gn * p.c_sn, p.c_dtype, v);
    }
  }
}

int launch_simt(const tb_gemm_args& a, cudaStream_t stream) {
  // The fused activation exists on the tensor-core path only; the output fan-out is honoured here as well.
  if (a.epilogue_op != TB_EPILOGUE_NONE) return TB_ERR_UNSUPPORTED;
  if (a.num_c_copies < 0 || a.num_c_copies > 7 || (a.num_c_copies > 0 && a.c_copies == nullptr)) return TB_ERR_INVALID;
  SimtParams p;
  p.M = a.m; p.N = a.n; p.K = a.k;
  p.A = a.a; p.a_sm = a.a_stride_m; p.a_sk = a.a_stride_k; p.a_dtype = a.a_dtype;
  p.B = a.b; p.b_sk = a.b_stride_k; p.b_sn = a.b_stride_n; p.b_dtype = a.b_dtype;
  p.C = a.c; p.c_sm = a.c_stride_m; p.c_sn = a.c_stride_n; p.c_dtype = a.c_dtype;
  p.num_c_extra = a.num_c_copies;
  for (int x = 0; x < 7; ++x) p.c_extra[x] = x < a.num_c_copies ? a.c_copies[x] : nullptr;
  p.a_scale = a.a_scale; p.b_scale = a.b_scale;
  p.bias = a.bias; p.bias_stride = a.bias_stride; p.bias_dtype = a.bias_dtype;
  dim3 grid((a.n + BN - 1) / BN, (a.m + BM - 1) / BM, 1);
  if (a.a_dtype == TB_DTYPE_I8 && a.b_dtype == TB_DTYPE_I8) simt_gemm_kernel<int><<<grid, 256, 0, stream>>>(p);
  else simt_gemm_kernel<float><<<grid, 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "simt_gemm_kernel launch");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

}  // namespace

int gemm_fp32_exact(const tb_gemm_args& a, cudaStream_t stream) { return launch_simt(a, stream); }

int gemm_generic_loader(const tb_gemm_args& a, const tb_config&, cudaStream_t stream, int*) { return launch_simt(a, stream); }

}  // namespace tb
