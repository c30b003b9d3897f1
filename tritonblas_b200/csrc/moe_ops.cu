// Memory-bound helpers on either side of the grouped MoE GEMMs (no reference counterpart; the reference has no MoE path):
//   swiglu:   out[r, j] = silu(h[r, j]) * h[r, F + j]            (h = [gate | up], fp32 math, one cast)
//   combine:  out[t, :] = sum_k w[t, k] * y[pos[t, k], :]        (top-k weighted sum of expert outputs, fp32 accumulate
//                                                                 in k order, one cast)
// Both stream their inputs once with 16-byte accesses: swiglu moves 6 bytes per output element, combine 2 * (topk + 1).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common_host.h"

namespace tb {
namespace {

template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __uint_as_float(u[j] << 16);
      v[2 * j + 1] = __uint_as_float(u[j] & 0xFFFF0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      u[j] = *reinterpret_cast<uint32_t*>(&t);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
  }
};
template <>
struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 w = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[j]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&v)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      __half2 t = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      u[j] = *reinterpret_cast<uint32_t*>(&t);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(u[0], u[1], u[2], u[3]);
  }
};

template <typename T>
__global__ void __launch_bounds__(256) swiglu_kernel(const T* __restrict__ h, long long h_stride, T* __restrict__ out,
                                                       long long out_stride, long long rows, int ffn) {
  const int vec_per_row = ffn / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i - r * vec_per_row) * 8;
    float g[8], u[8], o[8];
    Vec8<T>::load(h + r * h_stride + c, g);
    Vec8<T>::load(h + r * h_stride + ffn + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.0f + expf(-g[j])) * u[j];
    Vec8<T>::store(out + r * out_stride + c, o);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) combine_kernel(const T* __restrict__ y, long long y_stride,
                                                        const long long* __restrict__ pos, const float* __restrict__ w,
                                                        T* __restrict__ out, long long out_stride, int tokens, int topk,
                                                        int hidden) {
  const int vec_per_row = hidden / 8;
  const long long total = static_cast<long long>(tokens) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i - static_cast<long long>(t) * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < topk; ++k) {
      const long long src = pos[static_cast<long long>(t) * topk + k];
      const float wk = w[static_cast<long long>(t) * topk + k];
      float v[8];
      Vec8<T>::load(y + src * y_stride + c, v);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = fmaf(v[j], wk, acc[j]);
    }
    Vec8<T>::store(out + static_cast<long long>(t) * out_stride + c, acc);
  }
}

int grid_for(long long work_items) {
  long long blocks = (work_items + 255) / 256;
  const long long cap = 148LL * 8 * 8;
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

bool aligned16(const void* p, long long stride_elems) {
  return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && ((stride_elems * 2) & 15) == 0;
}

}  // namespace
}  // namespace tb

extern "C" int tb_swiglu(const void* h, int64_t h_row_stride, void* out, int64_t out_row_stride, int64_t rows, int32_t ffn,
                         int32_t dtype, void* stream) {
  if (h == nullptr || out == nullptr || rows < 0 || ffn <= 0 || (ffn % 8) != 0) return TB_ERR_INVALID;
  if (rows == 0) return TB_OK;
  if (!tb::aligned16(h, h_row_stride) || !tb::aligned16(out, out_row_stride) || ((ffn * 2) & 15) != 0) return TB_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = tb::grid_for(rows * (ffn / 8));
  if (dtype == TB_DTYPE_BF16)
    tb::swiglu_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h), h_row_stride,
                                                          static_cast<__nv_bfloat16*>(out), out_row_stride, rows, ffn);
  else if (dtype == TB_DTYPE_F16)
    tb::swiglu_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(h), h_row_stride, static_cast<__half*>(out),
                                                   out_row_stride, rows, ffn);
  else
    return TB_ERR_UNSUPPORTED;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "swiglu_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

extern "C" int tb_moe_combine(const void* y, int64_t y_row_stride, const int64_t* pos, const float* weights, void* out,
                              int64_t out_row_stride, int32_t tokens, int32_t topk, int32_t hidden, int32_t dtype,
                              void* stream) {
  if (y == nullptr || pos == nullptr || weights == nullptr || out == nullptr) return TB_ERR_INVALID;
  if (tokens < 0 || topk <= 0 || hidden <= 0 || (hidden % 8) != 0) return TB_ERR_INVALID;
  if (tokens == 0) return TB_OK;
  if (!tb::aligned16(y, y_row_stride) || !tb::aligned16(out, out_row_stride)) return TB_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = tb::grid_for(static_cast<long long>(tokens) * (hidden / 8));
  if (dtype == TB_DTYPE_BF16)
    tb::combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y), y_row_stride,
                                                           reinterpret_cast<const long long*>(pos), weights,
                                                           static_cast<__nv_bfloat16*>(out), out_row_stride, tokens, topk, hidden);
  else if (dtype == TB_DTYPE_F16)
    tb::combine_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(y), y_row_stride,
                                                    reinterpret_cast<const long long*>(pos), weights,
                                                    static_cast<__half*>(out), out_row_stride, tokens, topk, hidden);
  else
    return TB_ERR_UNSUPPORTED;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "combine_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

// ------------------------------------------------------------------------------------------------------------------
// Expert-parallel dispatch / combine over peer-mapped memory (NVLink / NVSwitch), replacing all-to-all collectives:
//   dispatch: row i of the send list (token src_token[i]) is written straight into the receive buffer of the rank that
//             owns its expert, at the row that rank's grouped GEMM expects (dest_row[i]); rows are 16-byte vector copies,
//             so every row crosses NVLink as one contiguous run.
//   combine:  out[t, :] = sum_k w[t, k] * y_{pair_rank[t,k]}[pair_row[t,k], :], reading the experts' outputs from the
//             owners' buffers with ordinary peer loads.
// Ordinary loads and stores only: no TMA, no multicast, no multimem on peer memory. The caller places barriers between
// the phases (rows landed before the GEMMs read them; outputs complete before they are combined).
namespace tb {
namespace {

struct PeerPtrs {
  void* p[8];
};

__global__ void __launch_bounds__(256) moe_dispatch_kernel(const uint4* __restrict__ x, long long x_stride_vec,
                                                             const long long* __restrict__ src_token,
                                                             const int* __restrict__ dest_rank,
                                                             const long long* __restrict__ dest_row, PeerPtrs peers,
                                                             long long dest_stride_vec, long long n, int vec_per_row,
                                                             long long capacity_rows, int* __restrict__ overflow, int topk) {
  // one warp per row
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; r < n; r += warps) {
    const long long row = dest_row[r];
    if (row < 0 || row >= capacity_rows) {  // a receive buffer too small for this routing: drop the row, tell the host
      if (lane == 0 && overflow != nullptr) atomicAdd(overflow, 1);
      continue;
    }
    // without a source list the i-th entry is the flattened (token, k) pair i: token i / topk
    const long long token = src_token != nullptr ? src_token[r] : r / topk;
    const uint4* src = x + token * x_stride_vec;
    uint4* dst = reinterpret_cast<uint4*>(peers.p[dest_rank[r]]) + row * dest_stride_vec;
    for (int v = lane; v < vec_per_row; v += 32) dst[v] = src[v];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) combine_peers_kernel(PeerPtrs y_peers, long long y_stride,
                                                              const int* __restrict__ pair_rank,
                                                              const long long* __restrict__ pair_row,
                                                              const float* __restrict__ w, T* __restrict__ out,
                                                              long long out_stride, int tokens, int topk, int hidden,
                                                              long long capacity_rows) {
  const int vec_per_row = hidden / 8;
  const long long total = static_cast<long long>(tokens) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i - static_cast<long long>(t) * vec_per_row) * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // Eight experts at a time: first all their indices, then all their rows (eight independent 16-byte loads in flight per
    // thread instead of one), then the sum in k order.
    for (int k0 = 0; k0 < topk; k0 += 8) {
      const T* src[8];
      float wk[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        src[j] = nullptr;
        wk[j] = 0.f;
        if (k0 + j < topk) {
          const long long f = static_cast<long long>(t) * topk + k0 + j;
          const long long prow = pair_row[f];
          // a pair whose row the dispatch dropped (beyond the owner's capacity) contributes nothing
          if (prow >= 0 && prow < capacity_rows) {
            src[j] = static_cast<const T*>(y_peers.p[pair_rank[f]]) + prow * y_stride + c;
            wk[j] = w[f];
          }
        }
      }
      float v[8][8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (src[j] != nullptr) {
          Vec8<T>::load(src[j], v[j]);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (src[j] != nullptr) {
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[j][i], wk[j], acc[i]);
        }
      }
    }
    Vec8<T>::store(out + static_cast<long long>(t) * out_stride + c, acc);
  }
}

}  // namespace
}  // namespace tb

extern "C" int tb_moe_dispatch_peers(const void* x, int64_t x_row_stride, const int64_t* src_token, const int32_t* dest_rank,
                                     const int64_t* dest_row, void* const* peer_bufs, int32_t num_peers,
                                     int64_t dest_row_stride, int64_t capacity_rows, int32_t* overflow_count, int64_t n,
                                     int32_t hidden, int32_t dtype, int32_t topk, void* stream) {
  if (x == nullptr || dest_rank == nullptr || dest_row == nullptr || peer_bufs == nullptr) return TB_ERR_INVALID;
  if (src_token == nullptr && topk < 1) return TB_ERR_INVALID;
  if (num_peers < 1 || num_peers > 8 || n < 0 || hidden <= 0 || (hidden % 8) != 0) return TB_ERR_INVALID;
  if (dtype != TB_DTYPE_BF16 && dtype != TB_DTYPE_F16) return TB_ERR_UNSUPPORTED;
  if (n == 0) return TB_OK;
  if (!tb::aligned16(x, x_row_stride) || ((dest_row_stride * 2) & 15) != 0) return TB_ERR_ALIGNMENT;
  tb::PeerPtrs peers = {};
  for (int i = 0; i < num_peers; ++i) {
    if ((reinterpret_cast<uintptr_t>(peer_bufs[i]) & 15) != 0) return TB_ERR_ALIGNMENT;
    peers.p[i] = peer_bufs[i];
  }
  long long blocks = (n + 7) / 8;  // 8 warps per block, one row per warp
  if (blocks > 148LL * 8 * 4) blocks = 148LL * 8 * 4;
  tb::moe_dispatch_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), x_row_stride / 8, reinterpret_cast<const long long*>(src_token), dest_rank,
      reinterpret_cast<const long long*>(dest_row), peers, dest_row_stride / 8, n, hidden / 8, capacity_rows, overflow_count,
      topk < 1 ? 1 : topk);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "moe_dispatch_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

namespace tb {
namespace {
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x, long long x_stride_vec,
                                                            const long long* __restrict__ src_row, uint4* __restrict__ out,
                                                            long long out_stride_vec, long long n, int vec_per_row) {
  // one warp per output row; rows are streamed once
  const int lane = threadIdx.x & 31;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5; r < n; r += warps) {
    const uint4* src = x + src_row[r] * x_stride_vec;
    uint4* dst = out + r * out_stride_vec;
    for (int v = lane; v < vec_per_row; v += 32) __stcs(dst + v, __ldg(src + v));
  }
}
}  // namespace
}  // namespace tb

extern "C" int tb_moe_gather_rows(const void* x, int64_t x_row_stride, const int64_t* src_row, void* out,
                                  int64_t out_row_stride, int64_t n, int32_t hidden, void* stream) {
  if (x == nullptr || src_row == nullptr || out == nullptr || n < 0 || hidden <= 0 || (hidden % 8) != 0) return TB_ERR_INVALID;
  if (n == 0) return TB_OK;
  if (!tb::aligned16(x, x_row_stride) || !tb::aligned16(out, out_row_stride)) return TB_ERR_ALIGNMENT;
  long long blocks = (n + 7) / 8;
  if (blocks > 148LL * 8 * 4) blocks = 148LL * 8 * 4;
  tb::gather_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), x_row_stride / 8, reinterpret_cast<const long long*>(src_row), static_cast<uint4*>(out),
      out_row_stride / 8, n, hidden / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "gather_rows_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

extern "C" int tb_moe_combine_peers(void* const* y_peers, int32_t num_peers, int64_t y_row_stride, const int32_t* pair_rank,
                                    const int64_t* pair_row, const float* weights, void* out, int64_t out_row_stride,
                                    int32_t tokens, int32_t topk, int32_t hidden, int32_t dtype, int64_t capacity_rows,
                                    void* stream) {
  if (y_peers == nullptr || pair_rank == nullptr || pair_row == nullptr || weights == nullptr || out == nullptr) return TB_ERR_INVALID;
  if (num_peers < 1 || num_peers > 8 || tokens < 0 || topk <= 0 || hidden <= 0 || (hidden % 8) != 0 || capacity_rows < 0) return TB_ERR_INVALID;
  if (tokens == 0) return TB_OK;
  if (((y_row_stride * 2) & 15) != 0 || !tb::aligned16(out, out_row_stride)) return TB_ERR_ALIGNMENT;
  tb::PeerPtrs peers = {};
  for (int i = 0; i < num_peers; ++i) {
    if ((reinterpret_cast<uintptr_t>(y_peers[i]) & 15) != 0) return TB_ERR_ALIGNMENT;
    peers.p[i] = y_peers[i];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = tb::grid_for(static_cast<long long>(tokens) * (hidden / 8));
  if (dtype == TB_DTYPE_BF16)
    tb::combine_peers_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(peers, y_row_stride, pair_rank,
                                                                 reinterpret_cast<const long long*>(pair_row), weights,
                                                                 static_cast<__nv_bfloat16*>(out), out_row_stride, tokens, topk, hidden,
                                                                 capacity_rows);
  else if (dtype == TB_DTYPE_F16)
    tb::combine_peers_kernel<__half><<<grid, 256, 0, st>>>(peers, y_row_stride, pair_rank,
                                                          reinterpret_cast<const long long*>(pair_row), weights,
                                                          static_cast<__half*>(out), out_row_stride, tokens, topk, hidden,
                                                          capacity_rows);
  else
    return TB_ERR_UNSUPPORTED;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "combine_peers_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

// ------------------------------------------------------------------------------------------------------------------
// Dispatch plan on the device: where every routed (token, k) pair goes. Two small kernels replace a sort, a histogram and
// a dozen index operations:
//   count: counts[e] = pairs of this rank routed to expert e (shared-memory histogram per block, one global add per
//          expert and block);
//   plan:  given the counts of every rank (counts_all[r][e], after the ranks exchanged them), expert e lives on rank
//          e / experts_per_rank; inside its owner's receive buffer the experts follow each other and inside an expert the
//          source ranks follow each other. A pair of this rank routed to e gets row
//              owner_off[e] + sum_{r < rank} counts_all[r][e] + (its position among this rank's pairs of e),
//          the position taken from a per-expert cursor (block-aggregated, so the order inside an expert is arbitrary;
//          every row is computed independently of its position and the combine step sums in k order, so the result
//          does not depend on it).
namespace tb {
namespace {

constexpr int kPlanThreads = 256;
constexpr int kPlanItems = 4;       // pairs per thread
constexpr int kPlanMaxExperts = 1024;

// Expert of pair f in placement order: `place` (or the identity) maps an expert id to its position in the sequence of
// experts as they are laid out over the ranks (position q lives on rank q / experts_per_rank as its local expert
// q % experts_per_rank). -1 for an id outside [0, E).
__device__ __forceinline__ int expert_of(const void* ids, int is64, long long f, const int* place, int E) {
  const long long e = is64 ? static_cast<const long long*>(ids)[f] : static_cast<long long>(static_cast<const int*>(ids)[f]);
  if (e < 0 || e >= E) return -1;
  return place != nullptr ? place[e] : static_cast<int>(e);
}

__global__ void __launch_bounds__(kPlanThreads) moe_count_kernel(const void* __restrict__ ids, int is64, long long n, int E,
                                                                  const int* __restrict__ place, int* __restrict__ counts) {
  __shared__ int hist[kPlanMaxExperts];
  for (int e = threadIdx.x; e < E; e += kPlanThreads) hist[e] = 0;
  __syncthreads();
  const long long base = static_cast<long long>(blockIdx.x) * kPlanThreads * kPlanItems;
#pragma unroll
  for (int i = 0; i < kPlanItems; ++i) {
    const long long f = base + i * kPlanThreads + threadIdx.x;
    if (f < n) {
      const int e = expert_of(ids, is64, f, place, E);
      if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPlanThreads)
    if (hist[e] != 0) atomicAdd(&counts[e], hist[e]);
}

__global__ void __launch_bounds__(kPlanThreads) moe_plan_kernel(const void* __restrict__ ids, int is64, long long n, int E,
                                                                 const int* __restrict__ place, int world, int rank,
                                                                 const int* __restrict__ counts_all,
                                                                 int* __restrict__ cursor, long long capacity,
                                                                 int* __restrict__ pair_rank, long long* __restrict__ pair_row,
                                                                 int* __restrict__ group_offsets, int* __restrict__ row_token,
                                                                 int topk) {
  __shared__ int total[kPlanMaxExperts];      // rows of expert e over all source ranks
  __shared__ long long dest[kPlanMaxExperts]; // first row of this rank's pairs of expert e in the owner's buffer
  __shared__ int hist[kPlanMaxExperts];
  __shared__ int block_base[kPlanMaxExperts];
  const int epr = E / world;
  for (int e = threadIdx.x; e < E; e += kPlanThreads) {
    int t = 0, lower = 0;
    for (int r = 0; r < world; ++r) {
      const int c = counts_all[r * E + e];
      t += c;
      if (r < rank) lower += c;
    }
    total[e] = t;
    hist[e] = lower;        // parked here until the owner offsets are known
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPlanThreads) {
    long long off = 0;
    for (int j = (e / epr) * epr; j < e; ++j) off += total[j];
    dest[e] = off + hist[e];
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    // row offsets of this rank's own experts, clamped to the receive buffer (rows beyond it are dropped by the dispatch)
    for (int j = threadIdx.x; j <= epr; j += kPlanThreads) {
      long long off = 0;
      for (int i = 0; i < j; ++i) off += total[rank * epr + i];
      group_offsets[j] = static_cast<int>(off < capacity ? off : capacity);
    }
  }
  for (int e = threadIdx.x; e < E; e += kPlanThreads) hist[e] = 0;
  __syncthreads();
  const long long base = static_cast<long long>(blockIdx.x) * kPlanThreads * kPlanItems;
  int ex[kPlanItems], local[kPlanItems];
#pragma unroll
  for (int i = 0; i < kPlanItems; ++i) {
    const long long f = base + i * kPlanThreads + threadIdx.x;
    ex[i] = -1;
    local[i] = 0;
    if (f < n) {
      const int e = expert_of(ids, is64, f, place, E);
      if (e >= 0 && e < E) {
        ex[i] = e;
        local[i] = atomicAdd(&hist[e], 1);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += kPlanThreads) block_base[e] = hist[e] != 0 ? atomicAdd(&cursor[e], hist[e]) : 0;
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kPlanItems; ++i) {
    const long long f = base + i * kPlanThreads + threadIdx.x;
    if (f < n) {
      const int e = ex[i];
      // an expert id outside [0, E) routes nowhere: row -1 is dropped by the dispatch and skipped by the combine
      const long long row = e >= 0 ? dest[e] + block_base[e] + local[i] : -1;
      pair_rank[f] = e >= 0 ? e / epr : 0;
      pair_row[f] = row;
      // single rank: the inverse map, source token of every row, for a grouped GEMM that gathers its rows by index
      if (row_token != nullptr && row >= 0 && row < capacity) row_token[row] = static_cast<int>(f / topk);
    }
  }
}

}  // namespace
}  // namespace tb

extern "C" int tb_moe_count(const void* topk_ids, int32_t ids_are_int64, int64_t n_pairs, int32_t num_experts,
                            const int32_t* expert_place, int32_t* counts, void* stream) {
  if (topk_ids == nullptr || counts == nullptr || n_pairs < 0 || num_experts < 1 || num_experts > tb::kPlanMaxExperts)
    return TB_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int32_t) * num_experts, st);
  if (e != cudaSuccess) return tb::cuda_fail(e, "cudaMemsetAsync(counts)");
  if (n_pairs == 0) return TB_OK;
  const long long per_block = tb::kPlanThreads * tb::kPlanItems;
  const unsigned blocks = static_cast<unsigned>((n_pairs + per_block - 1) / per_block);
  tb::moe_count_kernel<<<blocks, tb::kPlanThreads, 0, st>>>(topk_ids, ids_are_int64, n_pairs, num_experts, expert_place, counts);
  e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "moe_count_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

extern "C" int tb_moe_plan(const void* topk_ids, int32_t ids_are_int64, int64_t n_pairs, int32_t num_experts,
                           const int32_t* expert_place, int32_t world, int32_t rank, const int32_t* counts_all, int32_t* cursor, int64_t capacity_rows,
                           int32_t* pair_rank, int64_t* pair_row, int32_t* group_offsets, int32_t* row_token, int32_t topk,
                           void* stream) {
  if (topk_ids == nullptr || counts_all == nullptr || cursor == nullptr || pair_rank == nullptr || pair_row == nullptr ||
      group_offsets == nullptr)
    return TB_ERR_INVALID;
  if (n_pairs < 0 || num_experts < 1 || num_experts > tb::kPlanMaxExperts || world < 1 || rank < 0 || rank >= world ||
      (num_experts % world) != 0 || capacity_rows < 0 || (row_token != nullptr && (world != 1 || topk < 1)))
    return TB_ERR_INVALID;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(cursor, 0, sizeof(int32_t) * num_experts, st);
  if (e != cudaSuccess) return tb::cuda_fail(e, "cudaMemsetAsync(cursor)");
  const long long per_block = tb::kPlanThreads * tb::kPlanItems;
  const unsigned blocks = static_cast<unsigned>(n_pairs > 0 ? (n_pairs + per_block - 1) / per_block : 1);
  tb::moe_plan_kernel<<<blocks, tb::kPlanThreads, 0, st>>>(topk_ids, ids_are_int64, n_pairs, num_experts, expert_place, world, rank,
                                                          counts_all, cursor, capacity_rows, pair_rank,
                                                          reinterpret_cast<long long*>(pair_row), group_offsets, row_token,
                                                          topk < 1 ? 1 : topk);
  e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "moe_plan_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

// ------------------------------------------------------------------------------------------------------------------
// Diagnostic: how fast this GPU's SMs can store into a buffer (local, or a peer's mapped into this process) when every
// row is written as one contiguous run of `run_bytes` at a pitch of `pitch_bytes`, the pattern of an epilogue that pushes
// output tiles to other GPUs. The fused GEMM + all-gather and the MoE dispatch are bounded by this rate; the figure
// depends on the run length and hardly on the number of storing warps. No reference counterpart.
namespace tb {
namespace {
__global__ void peer_store_probe_kernel(uint4* dst, long long pitch_vec, int run_vec, long long rows, int passes) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const long long warp_id = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long nwarps = static_cast<long long>(gridDim.x) * warps_per_block;
  const int lanes_per_row = run_vec < 32 ? run_vec : 32;   // lanes that cover one row per store instruction
  const int rows_per_inst = 32 / lanes_per_row;
  const uint4 v = make_uint4(lane, blockIdx.x, 2, 3);
  for (int pass = 0; pass < passes; ++pass)
    for (long long r0 = warp_id * rows_per_inst; r0 < rows; r0 += nwarps * rows_per_inst) {
      const long long r = r0 + lane / lanes_per_row;
      if (r < rows)
        for (int c = lane % lanes_per_row; c < run_vec; c += lanes_per_row) dst[r * pitch_vec + c] = v;
    }
}
}  // namespace
}  // namespace tb

extern "C" int tb_peer_store_probe(void* dst, int64_t pitch_bytes, int32_t run_bytes, int64_t rows, int32_t blocks,
                                   int32_t threads, int32_t passes, void* stream) {
  if (dst == nullptr || rows <= 0 || passes < 1 || blocks < 1 || threads < 32 || threads > 1024 || (threads & 31)) return TB_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(dst) & 15) || (pitch_bytes & 15) || (run_bytes & 15) || run_bytes < 16 || run_bytes > pitch_bytes)
    return TB_ERR_ALIGNMENT;
  if (run_bytes < 512 && (512 % run_bytes) != 0) return TB_ERR_INVALID;   // whole rows per 32-lane store instruction
  tb::peer_store_probe_kernel<<<static_cast<unsigned>(blocks), static_cast<unsigned>(threads), 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(dst), pitch_bytes / 16, run_bytes / 16, rows, passes);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "peer_store_probe_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}
