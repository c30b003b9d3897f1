// MXFP4 block quantiser, optionally fused with a 32-point Hadamard rotation of every 32-element K block.
//
// Quantiser arithmetic follows the reference kernel bit for bit (include/tritonblas/utils.py:679-726):
//   amax of the block -> (bits + 0x200000) & 0xFF800000 (round up to a power of two when the mantissa is >= 1.75)
//   -> e = clamp(floor(log2(.)) - 2, -127, 127) -> q = x * 2^-e -> e2m1 by integer operations (denormal shift below
//   1.0, re-bias, round to nearest with ties away from zero, saturate at 6.0) -> two codes per byte, even element in
//   the low nibble; scale byte = e + 127. The code itself comes from the hardware fp32 -> e2m1 conversion, arranged to
//   reproduce that rounding exactly (see encode_e2m1x8).
// The rotation has no reference counterpart; its operation order is fixed so results are reproducible bit for bit:
//   fp32 butterflies with strides 1, 2, 4, 8, 16, each (a, b) -> (a + b, a - b), no fused multiply-add, then one fp32
//   multiply by 0.17677669529663687 (1/sqrt(32)).
//
// One thread owns one 32-element block: 64 bytes in (16-bit inputs), 16 code bytes + 1 scale byte out. Consecutive lanes
// own consecutive blocks of a row, so a warp reads 2 KB and writes 512 + 32 contiguous bytes. Pure HBM streaming:
// 2.53 bytes per input element for 16-bit inputs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common_host.h"

namespace tb {
namespace {

template <typename T>
__device__ __forceinline__ void load_block(const T* src, float (&v)[32]);

template <>
__device__ __forceinline__ void load_block<__nv_bfloat16>(const __nv_bfloat16* src, float (&v)[32]) {
  const uint4* p = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 w = __ldcs(p + i);  // streamed once
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[i * 8 + j * 2] = __uint_as_float(u[j] << 16);
      v[i * 8 + j * 2 + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
    }
  }
}
template <>
__device__ __forceinline__ void load_block<__half>(const __half* src, float (&v)[32]) {
  const uint4* p = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint4 w = __ldcs(p + i);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = *reinterpret_cast<const __half2*>(&u[j]);
      const float2 f = __half22float2(h);
      v[i * 8 + j * 2] = f.x;
      v[i * 8 + j * 2 + 1] = f.y;
    }
  }
}
template <>
__device__ __forceinline__ void load_block<float>(const float* src, float (&v)[32]) {
  const float4* p = reinterpret_cast<const float4*>(src);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 w = __ldcs(p + i);
    v[i * 4] = w.x;
    v[i * 4 + 1] = w.y;
    v[i * 4 + 2] = w.z;
    v[i * 4 + 3] = w.w;
  }
}

// Two fp32 values in one 64-bit register and the packed fp32 arithmetic of sm_100 (two independent IEEE operations per
// instruction, same rounding as the scalar forms): halves the instruction count of the butterflies below.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long p, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// Same operations in the same order as the scalar definition (strides 1, 2, 4, 8, 16, then the multiply): for strides
// below 16 the two halves v[0..15] and v[16..31] go through identical, independent butterflies, so element j and element
// j + 16 share a packed register and every packed instruction does one butterfly leg of each half.
__device__ __forceinline__ void hadamard32(float (&v)[32]) {
  unsigned long long p[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) p[j] = pack2(v[j], v[j + 16]);
#pragma unroll
  for (int stride = 1; stride < 16; stride <<= 1) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      if ((j & stride) == 0) {
        const unsigned long long a = p[j], b = p[j + stride];
        p[j] = add2(a, b);
        p[j + stride] = sub2(a, b);
      }
    }
  }
  const unsigned long long c2 = pack2(0.17677669529663687f, 0.17677669529663687f);
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float lo, hi;
    unpack2(p[j], lo, hi);
    // stride 16 pairs the two halves of a register; then both results take the final multiply together
    const unsigned long long r = mul2(pack2(__fadd_rn(lo, hi), __fsub_rn(lo, hi)), c2);
    unpack2(r, v[j], v[j + 16]);
  }
}

// Eight fp32 values (already divided by the block scale) -> eight e2m1 codes, v[0] in the lowest nibble.
// The reference's integer recipe is round-to-nearest with ties away from zero and saturation at 6.0. The hardware
// conversion rounds ties to even, so the lowest mantissa bit of every input is set first: an exact tie (whose low bits
// are zero) moves one ulp up and rounds away from zero, while no other value can reach or cross a tie by gaining one
// ulp (a tie has that bit clear). Signs, -0.0 and saturation behave as in the recipe.
__device__ __forceinline__ uint32_t encode_e2m1x8(const float (&v)[8]) {
  float a[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) a[i] = __uint_as_float(__float_as_uint(v[i]) | 1u);
  uint32_t r;
  asm("{\n\t.reg .b8 t0, t1, t2, t3;\n\t.reg .b16 h0, h1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 t3, %8, %7;\n\t"
      "mov.b16 h0, {t0, t1};\n\tmov.b16 h1, {t2, t3};\n\tmov.b32 %0, {h0, h1};\n\t}"
      : "=r"(r)
      : "f"(a[0]), "f"(a[1]), "f"(a[2]), "f"(a[3]), "f"(a[4]), "f"(a[5]), "f"(a[6]), "f"(a[7]));
  return r;
}

// Byte offset of the scale of (row, K block) in atom order [row / 128][block / 4][512].
__device__ __forceinline__ long long atom_offset(int row, int blk, int k_atoms) {
  return (static_cast<long long>(row >> 7) * k_atoms + (blk >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (blk & 3);
}

__global__ void __launch_bounds__(256) scales_to_atoms_kernel(const unsigned char* __restrict__ scales, long long row_stride,
                                                                 unsigned char* __restrict__ atoms, int rows, int kblocks,
                                                                 int k_atoms, int row_groups) {
  // One thread per 32-bit word of the output: row r, K blocks 4a .. 4a+3 (padding gets 127 = scale 1.0).
  const long long total = static_cast<long long>(row_groups) * k_atoms * 128;
  for (long long w = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; w < total;
       w += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int word = static_cast<int>(w & 127);
    const long long atom = w >> 7;
    const int a = static_cast<int>(atom % k_atoms);
    const int g = static_cast<int>(atom / k_atoms);
    const int row = g * 128 + (word & 3) * 32 + (word >> 2);
    uint32_t v = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int blk = a * 4 + j;
      const uint32_t b = (row < rows && blk < kblocks) ? scales[row * row_stride + blk] : 0x7Fu;
      v |= b << (8 * j);
    }
    reinterpret_cast<uint32_t*>(atoms)[w] = v;
  }
}

template <typename T, bool HADAMARD>
__global__ void __launch_bounds__(256) quant_mxfp4_kernel(const T* __restrict__ x, long long x_row_stride,
                                                            unsigned char* __restrict__ codes, long long codes_row_stride,
                                                            unsigned char* __restrict__ scales, long long scales_row_stride,
                                                            unsigned char* __restrict__ atoms, int k_atoms, int rows,
                                                            int blocks_per_row) {
  const long long total = static_cast<long long>(rows) * blocks_per_row;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / blocks_per_row);
    const int blk = static_cast<int>(idx - static_cast<long long>(row) * blocks_per_row);
    float v[32];
    load_block<T>(x + row * x_row_stride + blk * 32, v);
    if (HADAMARD) hadamard32(v);
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    // block exponent
    const uint32_t p2 = (__float_as_uint(amax) + 0x200000u) & 0xFF800000u;
    const int exp_field = static_cast<int>(p2 >> 23);
    int e = exp_field == 255 ? 127 : exp_field - 129;
    e = e < -127 ? -127 : (e > 127 ? 127 : e);
    // 2^-e as bits (2^-127 is the denormal 0x00400000)
    const float inv_scale = __uint_as_float(e == 127 ? 0x00400000u : static_cast<uint32_t>(127 - e) << 23);
    uint32_t packed[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float q[8];
      const unsigned long long inv2 = pack2(inv_scale, inv_scale);
#pragma unroll
      for (int i = 0; i < 8; i += 2) unpack2(mul2(pack2(v[w * 8 + i], v[w * 8 + i + 1]), inv2), q[i], q[i + 1]);
      packed[w] = encode_e2m1x8(q);
    }
    *reinterpret_cast<uint4*>(codes + row * codes_row_stride + blk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    const unsigned char sbyte = static_cast<unsigned char>((e + 127) & 0xFF);
    if (scales != nullptr) scales[row * scales_row_stride + blk] = sbyte;
    if (atoms != nullptr)  // the arrangement the block-scaled MMA's scale copy consumes (see atom_offset)
      atoms[atom_offset(row, blk, k_atoms)] = sbyte;
  }
}

template <typename T>
int launch(const void* x, long long xs, void* codes, long long cs, void* scales, long long ss, void* atoms, int rows, int k,
           int hadamard, int num_sms, cudaStream_t stream) {
  const int k_atoms = (k + 127) / 128;
  const int bpr = k / 32;
  const long long total = static_cast<long long>(rows) * bpr;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(num_sms) * 8 * 4;  // a few waves of 8 resident CTAs per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (hadamard)
    quant_mxfp4_kernel<T, true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const T*>(x), xs, static_cast<unsigned char*>(codes), cs, static_cast<unsigned char*>(scales), ss,
        static_cast<unsigned char*>(atoms), k_atoms, rows, bpr);
  else
    quant_mxfp4_kernel<T, false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const T*>(x), xs, static_cast<unsigned char*>(codes), cs, static_cast<unsigned char*>(scales), ss,
        static_cast<unsigned char*>(atoms), k_atoms, rows, bpr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "quant_mxfp4_kernel launch");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

}  // namespace
}  // namespace tb

extern "C" int tb_mxfp4_quant_atoms(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* codes,
                                    int64_t codes_row_stride, void* scales, int64_t scales_row_stride, void* atoms,
                                    int32_t hadamard, void* stream) {
  if (x == nullptr || codes == nullptr || (scales == nullptr && atoms == nullptr)) return TB_ERR_INVALID;
  if (rows < 0 || k < 0 || (k % 32) != 0) return TB_ERR_INVALID;
  if (rows == 0 || k == 0) return TB_OK;
  if (rows > 0x7FFFFFFF || k > 0x7FFFFFFF) return TB_ERR_INVALID;
  const int es = x_dtype == TB_DTYPE_F32 ? 4 : 2;
  // 16-byte vector accesses: rows of x and of the code array must start 16-byte aligned
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || ((x_row_stride * es) & 15) != 0) return TB_ERR_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) != 0 || (codes_row_stride & 15) != 0) return TB_ERR_ALIGNMENT;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess) return TB_ERR_NO_DEVICE;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int r = static_cast<int>(rows), kk = static_cast<int>(k);
  switch (x_dtype) {
    case TB_DTYPE_BF16:
      return tb::launch<__nv_bfloat16>(x, x_row_stride, codes, codes_row_stride, scales, scales_row_stride, atoms, r, kk, hadamard, sms, st);
    case TB_DTYPE_F16:
      return tb::launch<__half>(x, x_row_stride, codes, codes_row_stride, scales, scales_row_stride, atoms, r, kk, hadamard, sms, st);
    case TB_DTYPE_F32:
      return tb::launch<float>(x, x_row_stride, codes, codes_row_stride, scales, scales_row_stride, atoms, r, kk, hadamard, sms, st);
    default: return TB_ERR_UNSUPPORTED;
  }
}

extern "C" int tb_mxfp4_quant(const void* x, int32_t x_dtype, int64_t rows, int64_t k, int64_t x_row_stride, void* codes,
                              int64_t codes_row_stride, void* scales, int64_t scales_row_stride, int32_t hadamard,
                              void* stream) {
  if (scales == nullptr) return TB_ERR_INVALID;
  return tb_mxfp4_quant_atoms(x, x_dtype, rows, k, x_row_stride, codes, codes_row_stride, scales, scales_row_stride, nullptr,
                              hadamard, stream);
}

extern "C" int64_t tb_mxfp4_atoms_bytes(int64_t rows, int64_t k) {
  if (rows <= 0 || k <= 0) return 0;
  return ((rows + 127) / 128) * ((k + 127) / 128) * 512;
}

extern "C" int tb_mxfp4_scales_to_atoms(const void* scales, int64_t scales_row_stride, int64_t rows, int64_t k, void* atoms,
                                        void* stream) {
  if (scales == nullptr || atoms == nullptr || rows < 0 || k < 0 || (k % 32) != 0) return TB_ERR_INVALID;
  if (rows == 0 || k == 0) return TB_OK;
  if (rows > 0x7FFFFFFF || k > 0x7FFFFFFF) return TB_ERR_INVALID;
  const int groups = static_cast<int>((rows + 127) / 128), k_atoms = static_cast<int>((k + 127) / 128);
  const long long words = static_cast<long long>(groups) * k_atoms * 128;
  long long blocks = (words + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  tb::scales_to_atoms_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char*>(scales), scales_row_stride, static_cast<unsigned char*>(atoms), static_cast<int>(rows),
      static_cast<int>(k / 32), k_atoms, groups);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "scales_to_atoms_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}
