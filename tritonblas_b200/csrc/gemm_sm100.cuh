// Persistent, warp-specialised GEMM for sm_100a: TMA -> shared-memory ring -> tcgen05.mma -> TMEM -> epilogue.
//
// One kernel covers the dense family (fp16 / bf16 / tf32 / fp8 operands, all four operand layouts, data-parallel and
// stream-K scheduling, optional per-row x per-column scales and N-broadcast bias). Tile width, operand majors, stage
// count and the schedule are run-time values; only the MMA kind and the CTA-pair width are compile-time.
//
// Roles inside a CTA of 192 threads:
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocator + MMA issuer (one elected lane; in a CTA pair only the even CTA issues)
//   warps 2..5  epilogue: TMEM -> registers -> (stream-K fix-up) -> scale, bias, cast -> global. A TMEM load takes
//               several hundred clocks to return and a warp can only wait for all of its loads at once, so each warp
//               issues the loads of a 64-column run together before it waits.
// The accumulator is double-buffered in TMEM so the epilogue of one work item overlaps the main loop of the next.
//
// Semantics follow the reference kernels: tile order with GROUP_SIZE_M swizzle (kernels/stages/schedule.py:124-145),
// epilogue order scale -> bias -> cast -> masked store (kernels/stages/matrix_view.py:263-301), hybrid stream-K with
// fp32 partial tiles reduced by the tile owner in increasing program order (kernels/streamk_gemm.py:175-324).
#pragma once
#include <type_traits>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace tb {

constexpr int kTileM = 128;          // accumulator rows per CTA (TMEM lanes)
constexpr int kStageRowBytes = 128;  // one swizzle row: K extent of a stage in bytes for K-major operands
constexpr int kEpiWarps = 4;                         // one per TMEM lane quarter
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;    // producer + MMA + epilogue warps
constexpr int kEpiWarp0 = 2;                         // first epilogue warp
constexpr int kEpiRowPitch = 128;                    // bytes per row of an epilogue warp's staging buffer; the eight 16-byte
                                                     // pieces of a row are XOR-swizzled with the row index (no padding)
constexpr int kEpiStageBytes = kEpiWarps * 32 * kEpiRowPitch;
constexpr int kSchedDepth = 4;         // tile indices in flight between the fetching warp and the other roles
constexpr int kSfAtomBytes = 512;      // scale factors of 128 rows x 4 K blocks, laid out [32 rows][4 row quads][4 blocks]
constexpr int kSfGroupsB = 2;          // 128-row scale groups staged for B: tiles are 64, 128 or 192 columns wide and start
                                       // at a multiple of 64 (the MMA takes its scale columns from an even TMEM column),
                                       // so a tile touches at most two groups
template <int KIND>
constexpr int gemm_threads() { return kGemmThreads; }
constexpr int kATileBytes = kTileM * kStageRowBytes;  // 16 KB

enum : int { TB_F16 = 0, TB_BF16 = 1, TB_F32 = 2, TB_E4M3 = 3, TB_E5M2 = 4, TB_U8 = 5, TB_I8 = 7 };

struct GemmParams {
  int M, N, K;
  int block_n;       // accumulator width (columns), multiple of 32, <= 256. For a CTA pair: the pair's width.
  int n_halves;      // 1, or 2: a work tile is two accumulators side by side (2 * block_n columns) that share the A
                     // tile of every stage; both TMEM accumulator stages then belong to one tile (no cross-tile overlap)
  int num_k_blocks;  // ceil(K / k elements per stage)
  int k_per_stage;   // K elements per stage
  int glu;  // 1 (CTA pairs only): B's rows are [gate | up] halves of N rows each (per group). The even CTA stages
            // block_n / 2 gate rows and the odd CTA the matching up rows, so every accumulator holds gate values in its
            // first block_n / 2 columns and up values in the rest; C (N columns) receives silu(gate) * up
  int a_mn3d, b_mn3d;  // MN-major operand described by a 3-D tensor map [mn / atom][k][atom]: one copy per stage
  int k_serpentine;  // 1: odd work items of a program load their K blocks in descending order
  int tiles_m, tiles_n, group_m;
  int stages;
  int esize;       // operand element size in bytes
  int a_mn, b_mn;  // 1 if the operand is stored with M (resp. N) contiguous instead of K
  uint32_t idesc;  // tcgen05 instruction descriptor
  uint32_t tmem_cols;
  // output and epilogue
  void* c_extra[7];  // further destinations with C's shape and strides (peer GPUs' buffers mapped into this process);
  int num_c_extra;   // every tile is stored to C and to each of them with ordinary stores
  int c_extra_tile_limit;  // only tiles with index below this go to the further destinations (the caller pushes the rest)
  void* C;
  long long ldc_m, ldc_n;
  int c_dtype;
  const float* a_scale;  // (M,) or null
  const float* b_scale;  // (N,) or null
  const void* bias;      // (N,) or null
  long long bias_stride;
  int bias_dtype;
  int staged_f32;        // 1: fp32 output, unit column stride, 16-byte aligned rows, no extra destinations
  int staged_store;      // 1: 16-bit output, unit column stride, 16-byte aligned rows in every destination
  int bias_along_m;      // 1: bias indexed by row (set when the problem was transposed to C^T = B^T A^T)
  // schedule
  int dp_tiles;  // tiles [0, dp_tiles) are data-parallel: tile = program + i * programs
  int sk_tiles;  // tiles [dp_tiles, dp_tiles + sk_tiles) have their K iterations split evenly over all programs
  float* partials;   // [programs * CTAS][block_n][128] fp32
  unsigned* flags;   // [programs * CTAS]
  unsigned epoch;    // value that marks a partial as published for this launch
  // grouped (MoE) mode: group g owns rows [group_offsets[g], group_offsets[g+1]) of A and C and rows
  // [g * N, (g + 1) * N) of B; null for a plain GEMM
  // Dynamic tile schedule (the reference's work-stealing mode): two zero-initialised words, [0] = tiles handed out beyond
  // every program's first one, [1] = programs that have finished fetching. The last program to finish zeroes both, so
  // launches that follow each other on a stream need no reset in between. nullptr: static round-robin schedule.
  unsigned* tile_counter;
  const int* group_offsets;
  int num_groups;
  // Row gather for A (grouped launches of the GATHER instantiation): row r of the problem is row a_gather[r] of the
  // matrix the A tensor map describes (box = one row of a stage's K extent); negative entries and rows past a group's end
  // read as zero. Every lane of the producer warp fetches four rows per stage with one gather-mode TMA copy.
  const int* a_gather;
  // Operand that no earlier work of the stream still writes (weights): 1 = the operand of tensor map A, 2 = of B, 0 =
  // none. With programmatic dependent launch a CTA can start while the previous kernel of the stream drains; it then
  // fills its shared-memory ring with that operand before it waits for the previous kernel (single CTAs, static
  // schedules, plain 2-D / 3-D operand copies).
  int early_operand;
  // failure reporting
  int* status;
  unsigned long long timeout_ns;
  // block-scaled (MXFP4) operands: scale factors arrive through two extra tensor maps over the pre-arranged
  // ("atom") layout [128-row group][K atom of 128 elements][512 bytes]
  long long* debug_out;  // bit 1 of debug_flags: per-CTA cycle counters of each role are written here
  int debug_flags;  // test / measurement knobs (results are wrong when set): bit 0 = unused,
                    // bit 1 = per-role cycle counters, bit 2 = stream-K programs never publish their partial-tile flag
};

struct WorkItem {
  int tile, kb0, kb1;
  bool valid;
};

// Enumerates the work of one program: first its slice of the stream-K iteration space, then its data-parallel tiles.
struct WorkIter {
  int pid, nprog, nkb, dp_tiles, sk_tiles;
  int dp_next;
  long long it, it_end;
  __device__ WorkIter(const GemmParams& p, int pid_, int nprog_, int grouped_tiles = -1)
      : pid(pid_), nprog(nprog_), nkb(p.num_k_blocks), dp_tiles(grouped_tiles >= 0 ? grouped_tiles : p.dp_tiles),
        sk_tiles(grouped_tiles >= 0 ? 0 : p.sk_tiles) {
    dp_next = pid;
    range(pid, it, it_end);
  }
  __device__ void range(int q, long long& b, long long& e) const {
    const long long total = static_cast<long long>(sk_tiles) * nkb;
    const long long base = total / nprog, rem = total % nprog;
    b = q * base + (q < rem ? q : rem);
    e = b + base + (q < rem ? 1 : 0);
  }
  // The split tiles come first: a program's partial tile is then published early in the launch, and the owners' fix-ups
  // (flag, partial tiles from L2, store: several round trips to a memory system that every SM is loading) happen while
  // the whole tiles still stream, instead of standing at the end of the launch where nothing hides them.
  __device__ WorkItem next() {
    WorkItem w;
    if (it < it_end) {
      const int t = static_cast<int>(it / nkb);
      const long long tile_end = static_cast<long long>(t + 1) * nkb;
      const long long e = it_end < tile_end ? it_end : tile_end;
      w.tile = dp_tiles + t;
      w.kb0 = static_cast<int>(it - static_cast<long long>(t) * nkb);
      w.kb1 = static_cast<int>(e - static_cast<long long>(t) * nkb);
      w.valid = true;
      it = e;
      return w;
    }
    if (dp_next < dp_tiles) {
      w.tile = dp_next;
      w.kb0 = 0;
      w.kb1 = nkb;
      w.valid = true;
      dp_next += nprog;
      return w;
    }
    w.valid = false;
    w.tile = w.kb0 = w.kb1 = 0;
    return w;
  }
};

__device__ __forceinline__ void tile_coords_dims(int tile, int tiles_m, int tiles_n, int group_m, int& tm, int& tn) {
  const int width = group_m * tiles_n;
  const int group = tile / width;
  const int first_m = group * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = tile - group * width;
  tm = first_m + r % gsz;
  tn = r / gsz;
}
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tile, int& tm, int& tn) {
  tile_coords_dims(tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
}

// Where a tile sits: first row of the tile in A / C, one past the last valid row, first column, first row of B.
struct TileGeom {
  int m0, row_end, n0, b_row0;
};
// tile_prefix (shared memory, grouped mode only): tiles before group g, for g in [0, num_groups].
__device__ __forceinline__ TileGeom tile_geometry(const GemmParams& p, int tile, int tile_m, const int* tile_prefix) {
  TileGeom g;
  int tm, tn;
  if (p.group_offsets == nullptr) {
    tile_coords(p, tile, tm, tn);
    g.m0 = tm * tile_m;
    g.row_end = p.M;
    g.n0 = tn * (p.glu ? p.block_n / 2 : p.block_n * p.n_halves);
    g.b_row0 = g.n0;
    return g;
  }
  int lo = 0, hi = p.num_groups;  // last group whose prefix is <= tile
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (tile_prefix[mid] <= tile) lo = mid;
    else hi = mid;
  }
  const int* offs = tile_prefix + p.num_groups + 1;  // shared-memory copy of the row offsets
  const int row0 = offs[lo], row1 = offs[lo + 1];
  const int tiles_m = (row1 - row0 + tile_m - 1) / tile_m;
  tile_coords_dims(tile - tile_prefix[lo], tiles_m, p.tiles_n, p.group_m, tm, tn);
  g.m0 = row0 + tm * tile_m;
  g.row_end = row1;
  g.n0 = tn * (p.glu ? p.block_n / 2 : p.block_n * p.n_halves);
  g.b_row0 = lo * (p.glu ? 2 * p.N : p.N) + g.n0;
  return g;
}

__device__ __forceinline__ float load_as_float(const void* p, long long idx, int dtype) {
  switch (dtype) {
    case TB_F16: return __half2float(reinterpret_cast<const __half*>(p)[idx]);
    case TB_BF16: return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
    default: return reinterpret_cast<const float*>(p)[idx];
  }
}

// Store 32 consecutive columns of one output row. `v` holds fp32 values after scale and bias.
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, void* c_base, int row, int col0, const float (&v)[32]) {
  const int ncols = min(32, p.N - col0);
  if (ncols <= 0) return;
  if (p.c_dtype == TB_BF16 || p.c_dtype == TB_F16) {
    unsigned short* base = reinterpret_cast<unsigned short*>(c_base) + row * p.ldc_m + col0 * p.ldc_n;
    if (p.ldc_n == 1 && ncols == 32 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
      uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float lo = v[j * 8 + h * 2], hi = v[j * 8 + h * 2 + 1];
          if (p.c_dtype == TB_BF16) {
            __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
            w[h] = *reinterpret_cast<uint32_t*>(&t);
          } else {
            __half2 t = __floats2half2_rn(lo, hi);
            w[h] = *reinterpret_cast<uint32_t*>(&t);
          }
        }
        dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (j < ncols) {
          unsigned short bits;
          if (p.c_dtype == TB_BF16) {
            __nv_bfloat16 t = __float2bfloat16_rn(v[j]);
            bits = *reinterpret_cast<unsigned short*>(&t);
          } else {
            __half t = __float2half_rn(v[j]);
            bits = *reinterpret_cast<unsigned short*>(&t);
          }
          base[j * p.ldc_n] = bits;
        }
      }
    }
  } else if (p.c_dtype == TB_F32) {
    float* base = reinterpret_cast<float*>(c_base) + row * p.ldc_m + col0 * p.ldc_n;
    if (p.ldc_n == 1 && ncols == 32 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
      float4* dst = reinterpret_cast<float4*>(base);
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols) base[j * p.ldc_n] = v[j];
    }
  } else if (p.c_dtype == TB_I8) {  // int8 output: round to nearest even, saturate
    signed char* base = reinterpret_cast<signed char*>(c_base) + row * p.ldc_m + col0 * p.ldc_n;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) base[j * p.ldc_n] = static_cast<signed char>(__float2int_rn(fminf(fmaxf(v[j], -128.0f), 127.0f)));
  } else {  // fp8 e4m3 output, saturating
    unsigned char* base = reinterpret_cast<unsigned char*>(c_base) + row * p.ldc_m + col0 * p.ldc_n;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) base[j * p.ldc_n] = static_cast<unsigned char>(__nv_cvt_float_to_fp8(v[j], __NV_SATFINITE, __NV_E4M3));
  }
}

// Fast-path epilogue math for 32 columns of one row: scale -> bias -> cast to the 16-bit output type, then the 64 bytes
// go into this lane's staging row as four 16-byte pieces, XOR-swizzled with the row index.
template <int KIND, bool BF16, bool MATH>
__device__ __forceinline__ void pack_chunk(const GemmParams& p, const uint32_t (&r)[32], uint8_t* mine, int lane, int col0,
                                           int piece0, float a_s, int row, int row_end) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = (KIND == 4) ? __int2float_rn(static_cast<int>(r[j])) : __uint_as_float(r[j]);
  if constexpr (MATH) {
    if (p.a_scale != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= a_s;
    }
    if (p.b_scale != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= p.b_scale[col0 + j];
    }
    if (p.bias != nullptr) {
      if (p.bias_along_m) {
        const float bv = row < row_end ? load_as_float(p.bias, row * p.bias_stride, p.bias_dtype) : 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += bv;
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] += load_as_float(p.bias, (col0 + j) * p.bias_stride, p.bias_dtype);
      }
    }
  }
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if constexpr (BF16) {
      __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&t);
    } else {
      __half2 t = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
      w[j] = *reinterpret_cast<uint32_t*>(&t);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j)
    *reinterpret_cast<uint4*>(mine + (((piece0 + j) ^ (lane & 7)) << 4)) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
}

// Drain of one whole 128 x block_n accumulator to a 16-bit row-major C (block_n a multiple of 64), straight-line per
// 64-column run: two TMEM loads in flight, pack into the warp's staging rows, read back as 128-byte row runs, store.
// `release` hands the accumulator back to the MMA issuer; it is called once the last columns sit in registers.
// kFix (stream-K tile owners): the fp32 partial tiles of `fix_count` peers, `fix_stride` floats apart starting at
// fix_src (already offset to this thread's row), are added in that order before scale, bias and cast.
template <int KIND, bool kBf16, bool kMath, bool kExtra, bool kFix, typename Release>
__device__ __forceinline__ void fast_drain(const GemmParams& p, uint8_t* stg, uint32_t t_row, int nchunks, int lane, int q,
                                           int m0, int n0, int row, int row_end, float a_s, Release&& release_accumulator,
                                           const float* fix_src = nullptr, size_t fix_stride = 0, int fix_count = 0) {

  const int seg = lane & 7, sub = lane >> 3;
  uint8_t* mine = stg + lane * kEpiRowPitch;
  unsigned short* c_rows = reinterpret_cast<unsigned short*>(p.C) +
                           static_cast<long long>(m0 + q * 32 + sub) * p.ldc_m + n0 + seg * 8;
  const long long off_base = static_cast<long long>(m0 + q * 32 + sub) * p.ldc_m + n0 + seg * 8;
  const int rows_left = row_end - (m0 + q * 32 + sub);  // this lane stores rows it*4 < rows_left
  for (int c0 = 0; c0 < nchunks; c0 += 2) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(t_row + c0 * 32, r0);
    tmem_ld_32x32(t_row + (c0 + 1) * 32, r1);
    tmem_ld_wait(r0);
    tmem_ld_wait(r1);
    if (c0 + 2 >= nchunks) release_accumulator();  // the last columns sit in registers
    if constexpr (kFix) {
      float f0[32], f1[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        f0[j] = (KIND == 4) ? __int2float_rn(static_cast<int>(r0[j])) : __uint_as_float(r0[j]);
        f1[j] = (KIND == 4) ? __int2float_rn(static_cast<int>(r1[j])) : __uint_as_float(r1[j]);
      }
      for (int pp = 0; pp < fix_count; ++pp) {
        const float* src = fix_src + pp * fix_stride + static_cast<size_t>(c0 * 32) * kTileM;
#pragma unroll
        for (int j = 0; j < 32; ++j) f0[j] += __ldcg(src + j * kTileM);
#pragma unroll
        for (int j = 0; j < 32; ++j) f1[j] += __ldcg(src + (32 + j) * kTileM);
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        r0[j] = __float_as_uint(f0[j]);
        r1[j] = __float_as_uint(f1[j]);
      }
      pack_chunk<0, kBf16, kMath>(p, r0, mine, lane, n0 + c0 * 32, 0, a_s, row, row_end);
      pack_chunk<0, kBf16, kMath>(p, r1, mine, lane, n0 + c0 * 32 + 32, 4, a_s, row, row_end);
    } else {
      pack_chunk<KIND, kBf16, kMath>(p, r0, mine, lane, n0 + c0 * 32, 0, a_s, row, row_end);
      pack_chunk<KIND, kBf16, kMath>(p, r1, mine, lane, n0 + c0 * 32 + 32, 4, a_s, row, row_end);
    }
    __syncwarp();
    uint4 val[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int row_l = it * 4 + sub;
      val[it] = *reinterpret_cast<const uint4*>(stg + row_l * kEpiRowPitch + ((seg ^ (row_l & 7)) << 4));
    }
#pragma unroll
    for (int it = 0; it < 8; ++it)
      if (it * 4 < rows_left)
        *reinterpret_cast<uint4*>(c_rows + static_cast<long long>(it * 4) * p.ldc_m + c0 * 32) = val[it];
    if constexpr (kExtra) {
      for (int x = 0; x < p.num_c_extra; ++x) {
        unsigned short* e_rows = reinterpret_cast<unsigned short*>(p.c_extra[x]) + off_base + c0 * 32;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          // read the staged piece again rather than keep 32 registers live across this loop
          const int row_l = it * 4 + sub;
          const uint4 again = *reinterpret_cast<const uint4*>(stg + row_l * kEpiRowPitch + ((seg ^ (row_l & 7)) << 4));
          if (it * 4 < rows_left) *reinterpret_cast<uint4*>(e_rows + static_cast<long long>(it * 4) * p.ldc_m) = again;
        }
      }
    }
    __syncwarp();
  }
}

// The same for a row-major fp32 C (16-byte aligned rows, whole tiles): per 32 columns the lane's 128-byte row passes
// through the staging rows and leaves as full 128-byte runs.
template <int KIND, bool kMath, typename Release>
__device__ __forceinline__ void fast_drain_f32(const GemmParams& p, uint8_t* stg, uint32_t t_row, int nchunks, int lane, int q,
                                               int m0, int n0, int row, int row_end, float a_s, Release&& release_accumulator) {
  const int seg = lane & 7, sub = lane >> 3;
  uint8_t* mine = stg + lane * kEpiRowPitch;
  float* c_rows = reinterpret_cast<float*>(p.C) + static_cast<long long>(m0 + q * 32 + sub) * p.ldc_m + n0 + seg * 4;
  const int rows_left = row_end - (m0 + q * 32 + sub);
  for (int c = 0; c < nchunks; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait(r);
    if (c + 1 == nchunks) release_accumulator();
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (KIND == 4) ? __int2float_rn(static_cast<int>(r[j])) : __uint_as_float(r[j]);
    if constexpr (kMath) {
      const int col0 = n0 + c * 32;
      if (p.a_scale != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= a_s;
      }
      if (p.b_scale != nullptr) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= p.b_scale[col0 + j];
      }
      if (p.bias != nullptr) {
        if (p.bias_along_m) {
          const float bv = row < row_end ? load_as_float(p.bias, row * p.bias_stride, p.bias_dtype) : 0.0f;
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += bv;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += load_as_float(p.bias, (col0 + j) * p.bias_stride, p.bias_dtype);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<float4*>(mine + ((j ^ (lane & 7)) << 4)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    __syncwarp();
    float4 val[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int row_l = it * 4 + sub;
      val[it] = *reinterpret_cast<const float4*>(stg + row_l * kEpiRowPitch + ((seg ^ (row_l & 7)) << 4));
    }
#pragma unroll
    for (int it = 0; it < 8; ++it)
      if (it * 4 < rows_left) *reinterpret_cast<float4*>(c_rows + static_cast<long long>(it * 4) * p.ldc_m + c * 32) = val[it];
    __syncwarp();
  }
}

// Drain of a gate/up accumulator: `nchunks` x 32 gate columns at t_gate, the matching up columns at t_up; C receives
// silu(gate) * up (fp32 math, one cast), 16-bit row-major, whole 64-column runs. Same staging scheme as
// fast_drain. `release` hands the accumulator back once the last columns sit in registers.
template <bool kBf16, typename Release>
__device__ __forceinline__ void glu_drain(const GemmParams& p, uint8_t* stg, uint32_t t_gate, uint32_t t_up, int nchunks,
                                          int lane, int q, int m0, int n0, int row_end, Release&& release_accumulators) {
  const int seg = lane & 7, sub = lane >> 3;
  uint8_t* mine = stg + lane * kEpiRowPitch;
  unsigned short* c_rows =
      reinterpret_cast<unsigned short*>(p.C) + static_cast<long long>(m0 + q * 32 + sub) * p.ldc_m + n0 + seg * 8;
  const int rows_left = row_end - (m0 + q * 32 + sub);
  for (int c0 = 0; c0 < nchunks; c0 += 2) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t g[32], u[32];
      tmem_ld_32x32(t_gate + (c0 + half) * 32, g);
      tmem_ld_32x32(t_up + (c0 + half) * 32, u);
      tmem_ld_wait(g);
      tmem_ld_wait(u);
      if (half == 1 && c0 + 2 >= nchunks) release_accumulators();
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
        const float v0 = g0 / (1.0f + __expf(-g0)) * __uint_as_float(u[2 * j]);
        const float v1 = g1 / (1.0f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
        if constexpr (kBf16) {
          __nv_bfloat162 t = __floats2bfloat162_rn(v0, v1);
          w[j] = *reinterpret_cast<uint32_t*>(&t);
        } else {
          __half2 t = __floats2half2_rn(v0, v1);
          w[j] = *reinterpret_cast<uint32_t*>(&t);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(mine + (((half * 4 + j) ^ (lane & 7)) << 4)) =
            make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
    __syncwarp();
    uint4 val[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int row_l = it * 4 + sub;
      val[it] = *reinterpret_cast<const uint4*>(stg + row_l * kEpiRowPitch + ((seg ^ (row_l & 7)) << 4));
    }
#pragma unroll
    for (int it = 0; it < 8; ++it)
      if (it * 4 < rows_left)
        *reinterpret_cast<uint4*>(c_rows + static_cast<long long>(it * 4) * p.ldc_m + c0 * 32) = val[it];
    __syncwarp();
  }
}

// Stream-K owner of a split tile: finds the programs after `pid` whose slice starts inside the tile and waits (bounded)
// until each has published its partial tile. Returns one past the last such program, or -1 if a wait gave up.
// One lane per warp polls (128 polling threads per CTA would load L2 for nothing while the peers still compute); once it
// has seen a flag, every lane reads it once itself, which is its own acquire. Out of line for the same reason as below.
template <int CTAS>
__device__ __noinline__ int wait_for_peers(const unsigned* flags, unsigned epoch, int sk_tiles, int nkb, int dp_tiles, int tile,
                                           int pid, int nprog, int cta_rank, int lane, volatile int* abort_flag, int* status,
                                           unsigned long long timeout_ns) {
  const WaitCtx wctx{abort_flag, status, timeout_ns};
  int peer_end = pid + 1;
  const long long tile_end = static_cast<long long>(tile - dp_tiles + 1) * nkb;
  const long long total = static_cast<long long>(sk_tiles) * nkb;
  const long long base = total / nprog, rem = total % nprog;
  while (peer_end < nprog) {  // same split as WorkIter::range
    const long long b = peer_end * base + (peer_end < rem ? peer_end : rem);
    const long long e = b + base + (peer_end < rem ? 1 : 0);
    if (b >= tile_end || b >= e) break;
    ++peer_end;
  }
  bool ok = true;
  for (int pp = pid + 1; pp < peer_end && ok; ++pp) {
    const unsigned* flag = &flags[pp * CTAS + cta_rank];
    bool seen = true;
    if (lane == 0) seen = flag_wait(flag, epoch, wctx, TB_DEV_TIMEOUT_PEER_FLAG);
    ok = __shfl_sync(0xffffffffu, seen ? 1 : 0, 0) != 0;
    __syncwarp();
    if (ok) ok = flag_wait(flag, epoch, wctx, TB_DEV_TIMEOUT_PEER_FLAG);
  }
  ok = __all_sync(0xffffffffu, ok);
  return ok ? peer_end : -1;
}

// Stream-K owner with 32-column accumulators: the partial tiles of `count` peers (`stride` floats apart, `src` already
// offset to this thread's row) are added up in program order and the 32 sums parked in this lane's 128-byte staging row
// (16-byte pieces XOR-swizzled with the lane, like every use of that buffer). Out of line: its registers would
// otherwise weigh on the drains of every launch.
static __device__ __noinline__ void park_peer_partials(const float* src, int count, size_t stride, uint8_t* mine, int lane) {
  float pre[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) pre[j] = 0.0f;
  for (int pp = 0; pp < count; ++pp, src += stride) {
#pragma unroll
    for (int j = 0; j < 32; ++j) pre[j] += __ldcg(src + j * kTileM);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<float4*>(mine + ((j ^ (lane & 7)) << 4)) =
        make_float4(pre[4 * j], pre[4 * j + 1], pre[4 * j + 2], pre[4 * j + 3]);
}

template <int KIND, int CTAS, bool PROF = false, bool GATHER = false>
__global__ void __launch_bounds__(gemm_threads<KIND>(), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is what the 128-byte swizzle pattern and the matrix descriptors assume.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const int pid = (CTAS == 2) ? (blockIdx.x >> 1) : blockIdx.x;
  const int nprog = (CTAS == 2) ? (gridDim.x >> 1) : gridDim.x;

  const int bn_local = p.block_n / CTAS;  // B rows this CTA stages
  const int b_tile_bytes = bn_local * kStageRowBytes;
  // Block-scaled kinds append the stage's scale factors: two K atoms for this CTA's A rows, then two K atoms for each
  // of the two 128-row groups of B that can overlap the tile.
  const int sf_bytes = (KIND == 3) ? (2 + 2 * kSfGroupsB) * kSfAtomBytes : 0;
  const int nh = (KIND == 3) ? 1 : p.n_halves;  // B tiles (and accumulators) per work tile
  const int stage_bytes = (kATileBytes + nh * b_tile_bytes + sf_bytes + 1023) & ~1023;
  const int stages = p.stages;

  uint8_t* ring = smem;
  uint8_t* epi_stage = smem + static_cast<size_t>(stages) * stage_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + kEpiStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + stages;
  uint64_t* tmem_full = bars + 2 * stages;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* publish_bar = tmem_empty + 2;  // the four epilogue warps have all written their part of a partial tile
  // dynamic schedule: a queue of tile indices from the fetching warp (producer of the even CTA) to every other role
  uint64_t* sched_full = publish_bar + 1;               // [kSchedDepth], one arrival: the fetcher
  uint64_t* sched_empty = sched_full + kSchedDepth;     // [kSchedDepth], one arrival per consuming warp of the pair
  uint32_t* tmem_ptr_slot = reinterpret_cast<uint32_t*>(sched_empty + kSchedDepth);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_slot + 1);
  volatile int* sched_q = reinterpret_cast<volatile int*>(tmem_ptr_slot + 2);  // [kSchedDepth]
  int* tile_prefix = reinterpret_cast<int*>(tmem_ptr_slot + 2 + kSchedDepth);  // grouped mode: [num_groups + 1]

  WaitCtx wctx{abort_flag, p.status, p.timeout_ns};
  constexpr bool prof = PROF;  // measurement instantiation: per-role cycle counters written to debug_out

  // One stage's copies of one operand for a single CTA (called by one thread; the barrier already expects the bytes).
  const int a_atom = kStageRowBytes / p.esize;  // elements per 128-byte row
  const int mn_box_bytes = p.k_per_stage * kStageRowBytes;
  auto load_a_single = [&](uint8_t* sa, uint64_t* bar, int k0, int m0) {
    if (!p.a_mn) {
      tma_load_2d(sa, &tmap_a, bar, k0, m0);
    } else if (p.a_mn3d) {
      tma_load_3d(sa, &tmap_a, bar, 0, k0, m0 / a_atom);
    } else {
      for (int j = 0; j < kTileM / a_atom; ++j) tma_load_2d(sa + j * mn_box_bytes, &tmap_a, bar, m0 + j * a_atom, k0);
    }
  };
  auto load_b_single = [&](uint8_t* sb, uint64_t* bar, int k0, int n0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (h >= nh) break;
      uint8_t* sbh = sb + h * b_tile_bytes;
      const int nh0 = n0 + h * p.block_n;
      if (!p.b_mn) {
        tma_load_2d(sbh, &tmap_b, bar, k0, nh0);
      } else if (p.b_mn3d) {
        tma_load_3d(sbh, &tmap_b, bar, 0, k0, nh0 / a_atom);
      } else {
        for (int j = 0; j < bn_local / a_atom; ++j) tma_load_2d(sbh + j * mn_box_bytes, &tmap_b, bar, nh0 + j * a_atom, k0);
      }
    }
  };
  // Stages of this program's first work item whose early operand was requested before the dependency wait (thread 0
  // counts them; the producer warp picks the number up from its lane 0).
  int early_stages = 0;

  if (threadIdx.x == 0) {
    // measurement instantiation: wall-clock stamps (ns) of this CTA's phases in words 9..15 of its counter block
    if (prof && p.debug_out != nullptr) {
      p.debug_out[blockIdx.x * 16 + 9] = static_cast<long long>(global_timer_ns());
      p.debug_out[blockIdx.x * 16 + 11] = static_cast<long long>(sm_id());  // which SM the CTA ran on
    }
    *abort_flag = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], kEpiWarps * CTAS);  // one arrival per epilogue warp of every CTA that shares the accumulator
    }
    mbar_init(publish_bar, kEpiWarps);
    for (int i = 0; i < kSchedDepth; ++i) {
      mbar_init(&sched_full[i], 1);
      // consumers: MMA issuer + 4 epilogue warps in the even CTA, producer + 4 epilogue warps in the odd one
      mbar_init(&sched_empty[i], 5 * CTAS);
    }
    mbar_fence_init();
    // Everything above touched only shared memory. From here on global memory is read, which has to wait for the
    // previous kernel of the stream when this launch was allowed to start before that one finished; only an operand the
    // caller declared untouched by earlier work may be requested before that.
    griddep_launch_dependents();
    if constexpr (CTAS == 1 && !GATHER && KIND != 3) {
      if (p.early_operand != 0 && p.group_offsets == nullptr && p.tile_counter == nullptr) {
        prefetch_tmap(p.early_operand == 1 ? &tmap_a : &tmap_b);
        WorkIter wi0(p, blockIdx.x, gridDim.x, -1);
        const WorkItem w0 = wi0.next();
        if (w0.valid) {
          const TileGeom tg = tile_geometry(p, w0.tile, kTileM, tile_prefix);
          early_stages = min(stages, w0.kb1 - w0.kb0);
          for (int st = 0; st < early_stages; ++st) {
            uint8_t* sa = ring + static_cast<size_t>(st) * stage_bytes;
            const int k0 = (w0.kb0 + st) * p.k_per_stage;  // a program's first item walks K forwards
            mbar_arrive_expect_tx(&full_bar[st], static_cast<uint32_t>(kATileBytes + nh * b_tile_bytes));
            if (p.early_operand == 1) load_a_single(sa, &full_bar[st], k0, tg.m0);
            else load_b_single(sa + kATileBytes, &full_bar[st], k0, tg.b_row0);
          }
        }
      }
    }
    griddep_wait();
    if (prof && p.debug_out != nullptr) p.debug_out[blockIdx.x * 16 + 10] = static_cast<long long>(global_timer_ns());
    if (p.group_offsets != nullptr) {
      // tile_prefix[0 .. G] = tiles before each group, followed by a copy of the G + 1 row offsets. The copy is clamped to
      // [0, M] and made non-decreasing: offsets that describe more rows than A and C hold (a receive buffer sized below
      // the worst case) then lose their tail instead of sending loads and stores past the end of the buffers.
      int acc_tiles = 0;
      int* offs = tile_prefix + p.num_groups + 1;
      tile_prefix[0] = 0;
      int row0 = min(max(p.group_offsets[0], 0), p.M);
      offs[0] = row0;
      for (int g = 0; g < p.num_groups; ++g) {
        const int row1 = min(max(p.group_offsets[g + 1], row0), p.M);
        offs[g + 1] = row1;
        acc_tiles += ((row1 - row0 + kTileM * CTAS - 1) / (kTileM * CTAS)) * p.tiles_n;
        tile_prefix[g + 1] = acc_tiles;
        row0 = row1;
      }
    }
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc<CTAS>(tmem_ptr_slot, p.tmem_cols);
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_slot;
  const int grouped_tiles = p.group_offsets != nullptr ? tile_prefix[p.num_groups] : -1;
  constexpr int kPairTileM = kTileM * CTAS;

  const int acc_stride = p.block_n;  // TMEM columns per accumulator stage

  // ---- dynamic tile schedule -------------------------------------------------------------------------------------
  // Every program starts with tile `pid`; after that the fetching warp (the producer of the even CTA) takes tile indices
  // from a global counter and hands each one to the other roles of the CTA (pair) through a small shared-memory queue.
  // Programs that start late, because other kernels hold their SMs, simply take fewer tiles.
  const bool dyn = p.tile_counter != nullptr;
  const int dyn_tiles = grouped_tiles >= 0 ? grouped_tiles : p.dp_tiles;
  // A consuming role's next work item (whole tiles only). seq counts the items this role has taken.
  auto dyn_take = [&](int seq, bool& ok) -> WorkItem {
    const int slot = seq & (kSchedDepth - 1);
    const uint32_t parity = (seq / kSchedDepth) & 1u;
    ok = __all_sync(0xffffffffu, (CTAS == 2) ? mbar_wait_cluster(&sched_full[slot], parity, wctx, TB_DEV_TIMEOUT_TILE_QUEUE)
                                             : mbar_wait(&sched_full[slot], parity, wctx, TB_DEV_TIMEOUT_TILE_QUEUE));
    WorkItem w;
    w.tile = ok ? sched_q[slot] : -1;
    w.kb0 = 0;
    w.kb1 = p.num_k_blocks;
    w.valid = w.tile >= 0;
    __syncwarp();
    if (lane == 0 && ok) {  // the slot may be refilled once every consumer has read it
      if (CTAS == 1 || cta_rank == 0) mbar_arrive(&sched_empty[slot]);
      else mbar_arrive_remote(mapa_cluster(smem_u32(&sched_empty[slot]), 0));
    }
    return w;
  };
  // The fetching warp's next work item; it also publishes it. Called by the whole producer warp of the even CTA.
  auto dyn_fetch = [&](int seq, bool& ok) -> WorkItem {
    const int slot = seq & (kSchedDepth - 1);
    const uint32_t parity = ((seq / kSchedDepth) & 1u) ^ 1u;  // passes at once the first time round
    ok = mbar_wait_warp(&sched_empty[slot], parity, wctx, TB_DEV_TIMEOUT_TILE_QUEUE);
    int t = -1;
    if (lane == 0 && ok) {
      if (seq == 0) t = pid;
      else t = static_cast<int>(atomicAdd(p.tile_counter, 1u)) + nprog;
      if (t >= dyn_tiles) {
        t = -1;
        // Every program ends with exactly one failed fetch (or an empty first tile); the last one to get here leaves the
        // counters zeroed for the next launch.
        if (atomicAdd(p.tile_counter + 1, 1u) == static_cast<unsigned>(nprog - 1)) {
          p.tile_counter[0] = 0u;
          p.tile_counter[1] = 0u;
        }
      }
      sched_q[slot] = t;
      if constexpr (CTAS == 2) {
        st_shared_cluster_u32(mapa_cluster(smem_u32(const_cast<int*>(&sched_q[slot])), 1), static_cast<uint32_t>(t));
        mbar_arrive_remote(mapa_cluster(smem_u32(&sched_full[slot]), 1));
      }
      mbar_arrive(&sched_full[slot]);
    }
    t = __shfl_sync(0xffffffffu, t, 0);
    WorkItem w;
    w.tile = t;
    w.kb0 = 0;
    w.kb1 = p.num_k_blocks;
    w.valid = ok && t >= 0;
    return w;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp walks the schedule (warp-uniform control flow); one elected lane issues the copies.
    {
      WorkIter wi(p, pid, nprog, grouped_tiles);
      int s = 0, item = 0;
      uint32_t ph = 0;
      // In a pair, transaction bytes of both CTAs land on the even CTA's barrier, which expects the sum.
      const uint32_t expect = static_cast<uint32_t>(kATileBytes + nh * b_tile_bytes + sf_bytes) * CTAS;
      // first stages of the first item: barrier armed and one operand already on its way (see the prologue)
      int early_left = __shfl_sync(0xffffffffu, early_stages, 0);
      bool ok = true;
      long long prof_wait = 0, prof_t0 = clock64();
      int seq = 0;
      auto next_item = [&]() -> WorkItem {
        if (!dyn) return wi.next();
        bool got = true;
        const WorkItem w = (cta_rank == 0) ? dyn_fetch(seq, got) : dyn_take(seq, got);
        ++seq;
        if (!got) ok = false;
        return w;
      };
      for (WorkItem w = next_item(); w.valid && ok; w = next_item()) {
        const TileGeom tg = tile_geometry(p, w.tile, kPairTileM, tile_prefix);
        const int m0 = tg.m0 + static_cast<int>(cta_rank) * kTileM;
        // row of the B map; in gate/up mode the odd CTA's rows are the up projection's, N rows further down
        const int n0 = tg.b_row0 + static_cast<int>(cta_rank) * (p.glu ? p.N : bn_local);
        const int sf_n0 = tg.n0;
        // Every other work item walks its K range backwards: the A and B slices the previous item touched last are the
        // ones most likely still in L2 (the accumulation order of those items is reversed with it).
        const bool backwards = p.k_serpentine && (item & 1);
        ++item;
        int grow[4] = {-1, -1, -1, -1};   // GATHER: source rows of this lane's four A rows (-1: reads as zeros)
        if constexpr (GATHER) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = m0 + 4 * lane + j;
            if (r < tg.row_end) grow[j] = __ldg(p.a_gather + r);
          }
        }
        for (int it = w.kb0; it < w.kb1; ++it) {
          const int kb = backwards ? w.kb0 + w.kb1 - 1 - it : it;
          const long long pw0 = prof ? clock64() : 0;
          ok = mbar_wait_warp(&empty_bar[s], ph ^ 1, wctx, TB_DEV_TIMEOUT_SMEM_EMPTY);
          if (!ok) break;
          if (prof) prof_wait += clock64() - pw0;
          uint8_t* sa = ring + static_cast<size_t>(s) * stage_bytes;
          uint8_t* sb = sa + kATileBytes;
          const int k0 = kb * p.k_per_stage;
          if (elect_one()) {
            if constexpr (CTAS == 1) {
              if (early_left == 0) mbar_arrive_expect_tx(&full_bar[s], expect);
              if constexpr (GATHER) {
                // A: every lane fetches its four rows below
              } else if (early_left == 0 || p.early_operand != 1) {
                load_a_single(sa, &full_bar[s], k0, m0);
              }
              if (early_left == 0 || p.early_operand != 2) load_b_single(sb, &full_bar[s], k0, n0);
              if constexpr (KIND == 3) {
                uint8_t* sf = sb + b_tile_bytes;
                // scale tensor maps are [row group][K atom][128 words]; a box holds the stage's two K atoms
                tma_load_3d(sf, &tmap_sfa, &full_bar[s], 0, 2 * kb, m0 >> 7);
                for (int g = 0; g < kSfGroupsB; ++g)
                  tma_load_3d(sf + (2 + 2 * g) * kSfAtomBytes, &tmap_sfb, &full_bar[s], 0, 2 * kb,
                              (sf_n0 >> 7) + g);
              }
            } else {
              const uint32_t bar = mapa_cluster(smem_u32(&full_bar[s]), 0);
              if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[s], expect);
              if constexpr (GATHER) {
                // A: every lane fetches its four rows below
              } else if (!p.a_mn) {
                tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);
              } else if (p.a_mn3d) {
                tma_load_3d_pair(sa, &tmap_a, bar, 0, k0, m0 / a_atom);
              } else {
                for (int j = 0; j < kTileM / a_atom; ++j)
                  tma_load_2d_pair(sa + j * mn_box_bytes, &tmap_a, bar, m0 + j * a_atom, k0);
              }
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (h >= nh) break;
                uint8_t* sbh = sb + h * b_tile_bytes;
                const int nh0 = n0 + h * p.block_n;
                if (!p.b_mn) {
                  tma_load_2d_pair(sbh, &tmap_b, bar, k0, nh0);
                } else if (p.b_mn3d) {
                  tma_load_3d_pair(sbh, &tmap_b, bar, 0, k0, nh0 / a_atom);
                } else {
                  for (int j = 0; j < bn_local / a_atom; ++j)
                    tma_load_2d_pair(sbh + j * mn_box_bytes, &tmap_b, bar, nh0 + j * a_atom, k0);
                }
              }
              if constexpr (KIND == 3) {
                // Each CTA of the pair needs the scales of its own A rows and of every B row of the tile.
                uint8_t* sf = sb + b_tile_bytes;
                tma_load_3d_pair(sf, &tmap_sfa, bar, 0, 2 * kb, m0 >> 7);
                for (int g = 0; g < kSfGroupsB; ++g)
                  tma_load_3d_pair(sf + (2 + 2 * g) * kSfAtomBytes, &tmap_sfb, bar, 0, 2 * kb,
                                   (sf_n0 >> 7) + g);
              }
            }
          }
          __syncwarp();
          if constexpr (GATHER) {
            // Lane l owns rows 4 l .. 4 l + 3 of the A tile: one gather-mode copy of four rows of the source matrix,
            // 512 bytes, into its slot of the swizzled stage (the byte count expected above already includes them;
            // rows out of range arrive as zeros). Issued after the elected lane's expect_tx (the __syncwarp above).
            if constexpr (CTAS == 1)
              tma_gather4_2d(sa + lane * 4 * kStageRowBytes, &tmap_a, &full_bar[s], k0, grow[0], grow[1], grow[2], grow[3]);
            else
              tma_gather4_2d_pair(sa + lane * 4 * kStageRowBytes, &tmap_a, mapa_cluster(smem_u32(&full_bar[s]), 0), k0,
                                  grow[0], grow[1], grow[2], grow[3]);
          }
          if (early_left > 0) --early_left;
          if (++s == stages) {
            s = 0;
            ph ^= 1;
          }
        }
      }
      if (prof && p.debug_out != nullptr && lane == 0) {
        p.debug_out[blockIdx.x * 16 + 0] = prof_wait;
        p.debug_out[blockIdx.x * 16 + 1] = clock64() - prof_t0;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Warp-uniform loop; one elected lane issues the MMAs and commits. In a pair only the even CTA issues.
    if (cta_rank == 0) {
      WorkIter wi(p, pid, nprog, grouped_tiles);
      int s = 0;
      uint32_t ph = 0;
      int acc = 0;
      // Byte distances inside one operand tile (see make_smem_desc).
      const uint32_t mn_atom_stride = static_cast<uint32_t>(p.k_per_stage) * kStageRowBytes;
      const uint32_t a_lead = p.a_mn ? mn_atom_stride : 16u, b_lead = p.b_mn ? mn_atom_stride : 16u;
      // K advance per MMA (32 bytes of K): 32 bytes inside the swizzle row, or (32/esize) rows of 128 bytes.
      const uint32_t a_kstep = (p.a_mn ? (32u / p.esize) * kStageRowBytes : 32u) >> 4;
      const uint32_t b_kstep = (p.b_mn ? (32u / p.esize) * kStageRowBytes : 32u) >> 4;
      // MN-major 32-bit operands use the 32-byte-chunk swizzle, whose pattern repeats every 4 rows (512 bytes).
      const uint32_t a_type = (p.a_mn && p.esize == 4) ? 1u : 2u, b_type = (p.b_mn && p.esize == 4) ? 1u : 2u;
      const uint32_t a_sbo = a_type == 1u ? 512u : 1024u, b_sbo = b_type == 1u ? 512u : 1024u;
      const uint32_t ring_addr = smem_u32(ring);
      // Descriptors of stage 0; a stage adds stage_bytes >> 4 to the start-address field.
      const uint64_t adesc0 = make_smem_desc(ring_addr, a_lead, a_sbo, a_type);
      const uint64_t bdesc0 = make_smem_desc(ring_addr + kATileBytes, b_lead, b_sbo, b_type);
      const uint32_t stage_step = static_cast<uint32_t>(stage_bytes) >> 4;
      const uint32_t idesc = p.idesc;
      bool ok = true;
      long long prof_full = 0, prof_tmem = 0, prof_issue = 0, prof_t0 = clock64(), prof_first_full = 0;
      uint32_t acc_parity = 0u;  // bit a: parity of how often TMEM accumulator a has been handed to the epilogue
      // The four MMAs of one stage (32 bytes of K each) into one accumulator; called by the elected lane.
      auto issue_stage = [&](uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t first) {
        umma<KIND, CTAS>(d_tmem, adesc, bdesc, idesc, first);
        umma<KIND, CTAS>(d_tmem, adesc + a_kstep, bdesc + b_kstep, idesc, 1u);
        umma<KIND, CTAS>(d_tmem, adesc + 2 * a_kstep, bdesc + 2 * b_kstep, idesc, 1u);
        umma<KIND, CTAS>(d_tmem, adesc + 3 * a_kstep, bdesc + 3 * b_kstep, idesc, 1u);
      };
      auto commit = [&](uint64_t* bar) {
        if constexpr (CTAS == 1) umma_commit(bar);
        else umma_commit_pair(bar, 3);
      };
      // This warp runs alone on its scheduler, so every instruction and every taken branch of the per-stage loop is
      // exposed latency; the narrow and the wide tile therefore get a loop each, with nothing in it that can be
      // decided per work item.
      int seq = 0;
      auto next_item = [&]() -> WorkItem {
        if (!dyn) return wi.next();
        bool got = true;
        const WorkItem w = dyn_take(seq, got);
        ++seq;
        if (!got) ok = false;
        return w;
      };
      for (WorkItem w = next_item(); w.valid && ok; w = next_item()) {
        // One accumulator per work item, alternating (the epilogue of one item overlaps the next item's main loop), or
        // both accumulators for the two halves of a wide tile.
        const int acc0 = (nh == 2) ? 0 : acc;
        // the epilogue must have drained the accumulator before the first MMA of the item overwrites it
        const long long pt0 = PROF ? clock64() : 0;
        ok = mbar_wait_warp(&tmem_empty[acc0], ((acc_parity >> acc0) & 1u) ^ 1u, wctx, TB_DEV_TIMEOUT_TMEM_EMPTY);
        if (!ok) break;
        if (PROF) prof_tmem += clock64() - pt0;
        tc_fence_after();
        const uint32_t d0 = tmem_base + static_cast<uint32_t>(acc0 * acc_stride);
        if (nh == 1) {
          // Block-scaled kinds: where the tile's first column sits inside its first 128-row scale group.
          const int mma_n0 = (KIND == 3) ? tile_geometry(p, w.tile, kPairTileM, tile_prefix).n0 : 0;
          const uint32_t sfb_col0 = static_cast<uint32_t>(mma_n0 & 127) >> 5;
          const int sf_groups_used = ((mma_n0 & 127) + p.block_n + 127) >> 7;
          for (int kb = w.kb0; kb < w.kb1; ++kb) {
            const long long pf0 = PROF ? clock64() : 0;
            ok = mbar_wait_warp(&full_bar[s], ph, wctx, TB_DEV_TIMEOUT_SMEM_FULL);
            if (!ok) break;
            const long long pf1 = PROF ? clock64() : 0;
            if (PROF) prof_full += pf1 - pf0;
            if (PROF && prof_first_full == 0) prof_first_full = static_cast<long long>(global_timer_ns());
            const uint64_t soff = static_cast<uint64_t>(s * stage_step);
            const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
            const uint32_t first = (kb > w.kb0) ? 1u : 0u;
            if (elect_one()) {
              if constexpr (KIND == 3) {
                // Scale factors of this stage: shared memory -> TMEM (one buffer, rewritten every stage; the copies and
                // the MMAs that follow execute in issue order). TMEM columns, one per 32 rows:
                //   [A atom0 (4) | A atom1 (4) | B atom0: 2 groups (8) | B atom1: 2 groups (8)].
                const uint32_t sf_smem = ring_addr + static_cast<uint32_t>(s) * stage_bytes + kATileBytes + b_tile_bytes;
                const uint32_t sfa_t = tmem_base + 2u * acc_stride;
                const uint32_t sfb_t = sfa_t + 8u;
#pragma unroll
                for (int t = 0; t < 2; ++t)
                  tmem_cp_32x128b_warpx4<CTAS>(sfa_t + 4u * t, make_smem_desc_noswizzle(sf_smem + t * kSfAtomBytes, 16, 128));
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                  for (int g = 0; g < kSfGroupsB; ++g)
                    if (g < sf_groups_used)
                      tmem_cp_32x128b_warpx4<CTAS>(
                          sfb_t + 4u * (t * kSfGroupsB + g),
                          make_smem_desc_noswizzle(sf_smem + (2 + g * 2 + t) * kSfAtomBytes, 16, 128));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  // an MMA covers 64 K elements = two scale bytes: bytes {0,1} or {2,3} of the atom's columns
                  const uint32_t sf_id = (k & 1) * 2u;
                  const uint32_t id = idesc | (sf_id << 4) | (sf_id << 29);
                  umma_mxf4<CTAS>(d0, adesc + k * a_kstep, bdesc + k * b_kstep, id,
                                  (sfa_t + 4u * (k >> 1)) | (sf_id << 30),
                                  (sfb_t + 4u * (k >> 1) * kSfGroupsB + sfb_col0) | (sf_id << 30), k == 0 ? first : 1u);
                }
              } else {
                issue_stage(d0, adesc, bdesc, first);
              }
              commit(&empty_bar[s]);  // frees the stage once every MMA that reads it has finished
              if (kb + 1 == w.kb1) commit(&tmem_full[acc0]);
            }
            __syncwarp();
            if (PROF) prof_issue += clock64() - pf1;
            if (++s == stages) {
              s = 0;
              ph ^= 1;
            }
          }
          if (!ok) break;
          acc_parity ^= 1u << acc0;
          acc ^= 1;
        } else {
          // wide tile: accumulators 0 and 1 side by side, both fed from every stage's A tile
          const uint32_t d1 = tmem_base + static_cast<uint32_t>(acc_stride);
          const uint64_t half_off = static_cast<uint64_t>(b_tile_bytes >> 4);
          for (int kb = w.kb0; kb < w.kb1; ++kb) {
            const long long pf0 = PROF ? clock64() : 0;
            ok = mbar_wait_warp(&full_bar[s], ph, wctx, TB_DEV_TIMEOUT_SMEM_FULL);
            if (!ok) break;
            const long long pf1 = PROF ? clock64() : 0;
            if (PROF) prof_full += pf1 - pf0;
            const uint64_t soff = static_cast<uint64_t>(s * stage_step);
            const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
            const uint32_t first = (kb > w.kb0) ? 1u : 0u;
            const bool last = kb + 1 == w.kb1;
            if (elect_one()) {
              issue_stage(d0, adesc, bdesc, first);
              if (last) commit(&tmem_full[0]);
            }
            __syncwarp();
            if (kb == w.kb0) {
              // the second accumulator may still be draining while the first already takes this stage
              const long long pt1 = PROF ? clock64() : 0;
              ok = mbar_wait_warp(&tmem_empty[1], ((acc_parity >> 1) & 1u) ^ 1u, wctx, TB_DEV_TIMEOUT_TMEM_EMPTY);
              if (!ok) break;
              if (PROF) prof_tmem += clock64() - pt1;
              tc_fence_after();
            }
            if (elect_one()) {
              issue_stage(d1, adesc, bdesc + half_off, first);
              commit(&empty_bar[s]);
              if (last) commit(&tmem_full[1]);
            }
            __syncwarp();
            if (PROF) prof_issue += clock64() - pf1;
            if (++s == stages) {
              s = 0;
              ph ^= 1;
            }
          }
          if (!ok) break;
          acc_parity ^= 3u;
        }
      }
      if (prof && p.debug_out != nullptr && lane == 0) {
        p.debug_out[blockIdx.x * 16 + 12] = prof_first_full;
        p.debug_out[blockIdx.x * 16 + 13] = static_cast<long long>(global_timer_ns());
        p.debug_out[blockIdx.x * 16 + 2] = prof_full;
        p.debug_out[blockIdx.x * 16 + 3] = prof_tmem;
        p.debug_out[blockIdx.x * 16 + 4] = prof_issue;
        p.debug_out[blockIdx.x * 16 + 5] = clock64() - prof_t0;
      }
    }
  } else if (warp >= kEpiWarp0 && warp < kEpiWarp0 + kEpiWarps) {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const int row_in_tile = q * 32 + lane;
    uint8_t* stg = epi_stage + (warp - kEpiWarp0) * (32 * kEpiRowPitch);
    WorkIter wi(p, pid, nprog, grouped_tiles);
    int acc = 0;
    uint32_t epi_parity = 0u;  // bit a: parity of how often TMEM accumulator a has been drained
    const int slot = pid * CTAS + static_cast<int>(cta_rank);
    const size_t slot_elems = static_cast<size_t>(p.block_n) * kTileM;
    const uint32_t tmem_empty_remote = (CTAS == 2) ? mapa_cluster(smem_u32(&tmem_empty[0]), 0) : 0u;
    bool ok = true;
    long long prof_wait = 0, prof_t0 = clock64(), prof_drain = 0;
    int seq = 0;
    auto next_item = [&]() -> WorkItem {
      if (!dyn) return wi.next();
      bool got = true;
      const WorkItem w = dyn_take(seq, got);
      ++seq;
      if (!got) ok = false;
      return w;
    };
    for (WorkItem w = next_item(); w.valid && ok; w = next_item()) {
      const TileGeom tg = tile_geometry(p, w.tile, kPairTileM, tile_prefix);
      const int m0 = tg.m0 + static_cast<int>(cta_rank) * kTileM;
      const int row_end = tg.row_end;
      // A wide tile is two accumulators side by side: drain them one after the other.
      for (int h = 0; h < nh && ok; ++h) {
      const int acc_i = (nh == 2) ? h : acc;
      const int n0 = tg.n0 + h * p.block_n;
      const long long pe0 = prof ? clock64() : 0;
      const int row = m0 + row_in_tile;
      const bool owner = (w.kb0 == 0);
      const bool complete = owner && (w.kb1 == p.num_k_blocks);
      // Peers that hold the rest of this tile's K range: programs after this one whose slice starts inside the tile.
      // Single CTAs wait for their partial tiles while this program's own share of the tile is still being accumulated:
      // a peer's share of the tile is the first thing it does after its whole tiles, so the flags are normally set long
      // before, and the round trips to L2 (a microsecond each while every SM streams) stay off the end of the launch.
      int peer_end = pid + 1;
      // 32-column accumulators (the decode orientation): the peers' partial tiles, summed in program order, are fetched
      // early as well and parked in this lane's 128-byte row of the staging buffer, which is idle until the drain
      const bool prefetch_fix = CTAS == 1 && owner && !complete && p.block_n == 32;
      // Only where the early fetch applies is the wait moved ahead of the accumulator's: elsewhere it measured 2 % slower
      // (M = 128, 256-column tiles), and in the pair instantiation the order cost the main drain registers.
      if constexpr (CTAS == 1) {
        if (prefetch_fix) {
          peer_end = wait_for_peers<CTAS>(p.flags, p.epoch, p.sk_tiles, p.num_k_blocks, p.dp_tiles, w.tile, pid, nprog,
                                          static_cast<int>(cta_rank), lane, abort_flag, p.status, p.timeout_ns);
          ok = peer_end >= 0;
          if (!ok) break;
          park_peer_partials(p.partials + static_cast<size_t>(pid + 1) * slot_elems + row_in_tile, peer_end - pid - 1,
                             slot_elems, stg + lane * kEpiRowPitch, lane);
        }
      }
      // Every decision to unwind is made warp-uniform: the TMEM loads below need the whole warp.
      ok = __all_sync(0xffffffffu, mbar_wait(&tmem_full[acc_i], (epi_parity >> acc_i) & 1u, wctx, TB_DEV_TIMEOUT_TMEM_FULL));
      if (!ok) break;
      if (prof) prof_wait += clock64() - pe0;
      tc_fence_after();
      if (owner && !complete && !prefetch_fix) {
        peer_end = wait_for_peers<CTAS>(p.flags, p.epoch, p.sk_tiles, p.num_k_blocks, p.dp_tiles, w.tile, pid, nprog,
                                        static_cast<int>(cta_rank), lane, abort_flag, p.status, p.timeout_ns);
        ok = peer_end >= 0;
        if (!ok) break;
      }

      const float a_s = (p.a_scale != nullptr && row < row_end) ? p.a_scale[row] : 1.0f;
      const int nchunks = p.block_n / 32;
      // further destinations of this tile (the tiles of a launch's tail may be left to a copy that follows the launch)
      const int n_extra = w.tile < p.c_extra_tile_limit ? p.num_c_extra : 0;
      // staged stores need whole 32-column chunks inside N and 16-byte aligned rows in every destination (host-checked)
      const bool staged = owner && p.staged_store && (n0 + p.block_n <= p.N);
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc_i * acc_stride);
      // Hand the accumulator back to the MMA issuer: called once the last chunk sits in registers, before it is stored.
      auto release_accumulator = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTAS == 1) mbar_arrive(&tmem_empty[acc_i]);
          else mbar_arrive_remote(tmem_empty_remote + acc_i * 8);
        }
      };
      if (p.glu) {
        // gate values in the accumulator's first block_n / 2 columns, up values in the rest: one fused drain of
        // block_n / 2 output columns (the host guarantees whole tiles of a data-parallel launch and a 16-bit row-major C)
        if (p.c_dtype == TB_BF16)
          glu_drain<true>(p, stg, t_row, t_row + p.block_n / 2, p.block_n / 64, lane, q, m0, tg.n0, row_end, release_accumulator);
        else
          glu_drain<false>(p, stg, t_row, t_row + p.block_n / 2, p.block_n / 64, lane, q, m0, tg.n0, row_end, release_accumulator);
      } else if (owner && staged && (p.block_n & 63) == 0 && (complete || n_extra == 0)) {
        // Common case (whole tile or a stream-K owner's fix-up, 16-bit row-major output, tile width a multiple of 64).
        // Every taken branch inside the drain loop costs an instruction refetch, and a handful of them per 64 columns is
        // what made a drain through the general path three to four times slower than its loads and stores take; so the
        // loop is straight-line, and the choices (output type, scales or bias, extra destinations, partial tiles to add)
        // are made once per tile by picking one of its instantiations.
        const bool has_math = p.a_scale != nullptr || p.b_scale != nullptr || p.bias != nullptr;
        const long long q0 = prof ? clock64() : 0;
        const float* fix_src =
            complete ? nullptr
                     : p.partials + static_cast<size_t>((pid + 1) * CTAS + static_cast<int>(cta_rank)) * slot_elems + row_in_tile;
#define TB_FAST_DRAIN(BF, MATH, EXTRA, FIX)                                                                      \
  fast_drain<KIND, BF, MATH, EXTRA, FIX>(p, stg, t_row, nchunks, lane, q, m0, n0, row, row_end, a_s, release_accumulator, \
                                         fix_src, static_cast<size_t>(CTAS) * slot_elems, peer_end - pid - 1)
        if (!complete) {
          if (p.c_dtype == TB_BF16) { if (has_math) TB_FAST_DRAIN(true, true, false, true); else TB_FAST_DRAIN(true, false, false, true); }
          else { if (has_math) TB_FAST_DRAIN(false, true, false, true); else TB_FAST_DRAIN(false, false, false, true); }
        } else if (n_extra > 0) {
          if (p.c_dtype == TB_BF16) { if (has_math) TB_FAST_DRAIN(true, true, true, false); else TB_FAST_DRAIN(true, false, true, false); }
          else { if (has_math) TB_FAST_DRAIN(false, true, true, false); else TB_FAST_DRAIN(false, false, true, false); }
        } else if (p.c_dtype == TB_BF16) {
          if (has_math) TB_FAST_DRAIN(true, true, false, false); else TB_FAST_DRAIN(true, false, false, false);
        } else {
          if (has_math) TB_FAST_DRAIN(false, true, false, false); else TB_FAST_DRAIN(false, false, false, false);
        }
#undef TB_FAST_DRAIN
        if (prof) prof_drain += clock64() - q0;
      } else if (complete && p.staged_f32 && n0 + p.block_n <= p.N) {
        if (p.a_scale != nullptr || p.b_scale != nullptr || p.bias != nullptr)
          fast_drain_f32<KIND, true>(p, stg, t_row, nchunks, lane, q, m0, n0, row, row_end, a_s, release_accumulator);
        else
          fast_drain_f32<KIND, false>(p, stg, t_row, nchunks, lane, q, m0, n0, row, row_end, a_s, release_accumulator);
      } else if (!owner) {
        // Partial tile of a stream-K launch: raw fp32 accumulators to this program's slot, column-major so that a warp
        // writes 128 contiguous bytes per column. The tile's owner is waiting for it, so this loop is kept straight-line.
        float* dst0 = p.partials + slot * slot_elems + row_in_tile;
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait(r);
          if (c + 1 == nchunks) release_accumulator();
          float* dst = dst0 + static_cast<size_t>(c * 32) * kTileM;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            dst[j * kTileM] = (KIND == 4) ? __int2float_rn(static_cast<int>(r[j])) : __uint_as_float(r[j]);
        }
      } else {
        // General path: fix-ups and whole tiles with any other output type or layout.
        for (int c = 0; c < nchunks; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + c * 32, r);
          tmem_ld_wait(r);
          if (c + 1 == nchunks) release_accumulator();
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j)
            v[j] = (KIND == 4) ? __int2float_rn(static_cast<int>(r[j])) : __uint_as_float(r[j]);  // int8 kind: int32 sums
          if (!owner) {
            // Publish a partial tile: column-major inside the slot so that a warp writes 128 contiguous bytes.
            float* dst = p.partials + slot * slot_elems + static_cast<size_t>(c * 32) * kTileM + row_in_tile;
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[j * kTileM] = v[j];
            continue;
          }
          if (prefetch_fix) {
            const uint8_t* mine = stg + lane * kEpiRowPitch;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 t = *reinterpret_cast<const float4*>(mine + ((j ^ (lane & 7)) << 4));
              v[4 * j] += t.x;
              v[4 * j + 1] += t.y;
              v[4 * j + 2] += t.z;
              v[4 * j + 3] += t.w;
            }
          } else {
            for (int pp = pid + 1; pp < peer_end; ++pp) {
              const float* src = p.partials + (pp * CTAS + static_cast<int>(cta_rank)) * slot_elems +
                                 static_cast<size_t>(c * 32) * kTileM + row_in_tile;
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += __ldcg(src + j * kTileM);
            }
          }
          const int col0 = n0 + c * 32;
          if (col0 < p.N && (staged || row < row_end)) {
            if (p.a_scale != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= a_s;
            }
            if (p.b_scale != nullptr) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= (col0 + j < p.N) ? p.b_scale[col0 + j] : 1.0f;
            }
            if (p.bias != nullptr) {
              if (p.bias_along_m) {
                const float bv = row < row_end ? load_as_float(p.bias, row * p.bias_stride, p.bias_dtype) : 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += bv;
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < p.N) v[j] += load_as_float(p.bias, (col0 + j) * p.bias_stride, p.bias_dtype);
              }
            }
            if (!staged) {
              store_row_chunk(p, p.C, row, col0, v);
              for (int x = 0; x < n_extra; ++x) store_row_chunk(p, p.c_extra[x], row, col0, v);
            }
          }
          if (staged) {
            // 16-bit outputs with unit column stride: the warp's 32 rows x 64 columns pass through shared memory so that
            // every row leaves as one 128-byte run (8 lanes x 16 bytes), which is what remote (NVLink) and local L2 writes
            // both want, instead of 16-byte pieces of 32 different rows per store instruction.
            uint8_t* mine = stg + lane * kEpiRowPitch;
            const int piece0 = (c & 1) * 4;
            uint32_t w[16];
            if (p.c_dtype == TB_BF16) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                __nv_bfloat162 t = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&t);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                __half2 t = __floats2half2_rn(v[2 * j], v[2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&t);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(mine + (((piece0 + j) ^ (lane & 7)) << 4)) =
                  make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
            if ((c & 1) || c + 1 == nchunks) {
              __syncwarp();
              const int ncol = (c & 1) ? 64 : 32;
              const int colw = n0 + (c & ~1) * 32;  // first column of the staged run
              const int seg = lane & 7;
              if (seg * 8 < ncol) {
                uint4 val[8];
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const int row_l = it * 4 + (lane >> 3);
                  val[it] = *reinterpret_cast<const uint4*>(stg + row_l * kEpiRowPitch + ((seg ^ (row_l & 7)) << 4));
                }
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const int row_g = m0 + q * 32 + it * 4 + (lane >> 3);
                  if (row_g < row_end) {
                    const long long off = static_cast<long long>(row_g) * p.ldc_m + colw + seg * 8;
                    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.C) + off) = val[it];
                    for (int x = 0; x < n_extra; ++x)
                      *reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.c_extra[x]) + off) = val[it];
                  }
                }
              }
              __syncwarp();
            }
          }
        }
      }
      if (!owner) {
        // A program publishes at most one partial tile per launch (only its first stream-K segment can start
        // inside a tile), so this barrier is used for a single phase.
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(publish_bar);
        if (warp == kEpiWarp0 && lane == 0) {
          // debug bit 2 (value 4) withholds the flag: the failure-path test uses it to make the owner's bounded wait run out
          if (mbar_wait(publish_bar, 0, wctx, TB_DEV_TIMEOUT_STORE) && !(p.debug_flags & 4)) flag_release(&p.flags[slot], p.epoch);
        }
      }
      epi_parity ^= 1u << acc_i;
      }  // halves
      if (nh == 1) acc ^= 1;
    }
    if (prof && p.debug_out != nullptr && threadIdx.x == kEpiWarp0 * 32) {
      p.debug_out[blockIdx.x * 16 + 14] = static_cast<long long>(global_timer_ns());
      p.debug_out[blockIdx.x * 16 + 6] = prof_wait;
      p.debug_out[blockIdx.x * 16 + 7] = clock64() - prof_t0;
      p.debug_out[blockIdx.x * 16 + 8] = prof_drain;
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // A wait gave up: let copies and MMAs already in flight land before shared memory and TMEM are released.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, p.tmem_cols);
  }
  if (prof && p.debug_out != nullptr && threadIdx.x == 0) p.debug_out[blockIdx.x * 16 + 15] = static_cast<long long>(global_timer_ns());
}

}  // namespace tb
