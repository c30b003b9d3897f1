// Copy of output tiles from this GPU's C into the same place of peer GPUs' buffers (mapped into this process), for the tail
// of a GEMM launch whose epilogue pushed only its first tiles: the launch then ends without waiting for the link, and this
// copy runs beside the next launch (on another stream), so the transfer of one product's last tiles overlaps the next
// product's first tiles, which have nothing to send yet. Ordinary loads and stores; tile order as the GEMM kernel's
// (GROUP_SIZE_M swizzle). No reference counterpart.
#include "common_host.h"

namespace tb {
namespace {

struct PushPeers {
  void* p[7];
};

__global__ void __launch_bounds__(256) push_tiles_kernel(const unsigned char* __restrict__ c, PushPeers peers, int n_peers,
                                                           long long pitch_bytes, int m, long long n_bytes, int tile_m,
                                                           int tile_n_bytes, int tiles_m, int tiles_n, int group_m,
                                                           int first_tile, int parts) {
  const int tile = first_tile + static_cast<int>(blockIdx.x) / parts;
  const int part = static_cast<int>(blockIdx.x) % parts;
  // tile -> (tm, tn), as tile_coords_dims of the GEMM kernel
  const int width = group_m * tiles_n;
  const int group = tile / width;
  const int first_m = group * group_m;
  const int gsz = min(tiles_m - first_m, group_m);
  const int r = tile - group * width;
  const int tm = first_m + r % gsz, tn = r / gsz;
  const int rows_per_part = tile_m / parts;
  const int row0 = tm * tile_m + part * rows_per_part;
  const int row1 = min(row0 + rows_per_part, m);
  const long long col0 = static_cast<long long>(tn) * tile_n_bytes;
  const int vecs = static_cast<int>((min(col0 + tile_n_bytes, n_bytes) - col0) >> 4);   // 16-byte pieces per row of the tile
  if (vecs <= 0) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  // Four rows per warp and pass: four independent 16-byte loads in flight per lane before any store is issued.
  for (int row = row0 + warp * 4; row < row1; row += warps * 4) {
    for (int v = lane; v < vecs; v += 32) {
      uint4 val[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (row + j < row1) val[j] = __ldcg(reinterpret_cast<const uint4*>(c + (row + j) * pitch_bytes + col0) + v);
      for (int x = 0; x < n_peers; ++x) {
        unsigned char* dst = static_cast<unsigned char*>(peers.p[x]);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (row + j < row1) reinterpret_cast<uint4*>(dst + (row + j) * pitch_bytes + col0)[v] = val[j];
      }
    }
  }
}

}  // namespace

int launch_push_tiles(const void* c, void* const* peers, int n_peers, long long pitch_bytes, int m, long long n_bytes, int tile_m,
                      int tile_n_bytes, int tiles_m, int tiles_n, int group_m, int first_tile, int num_tiles,
                      cudaStream_t stream) {
  if (num_tiles <= 0 || n_peers <= 0) return TB_OK;
  PushPeers pp = {};
  for (int x = 0; x < n_peers; ++x) pp.p[x] = peers[x];
  const int parts = 4;   // blocks per tile: 64 rows each for a 256-row tile
  // Launched beside a persistent GEMM (another stream) its CTAs share SMs with the GEMM's: measured on 4 GPUs the copy then
  // runs at half its stand-alone rate (0.31 against 0.166 ms for a 33.5 MB block to three peers) and the GEMM a fifth
  // slower; keeping it off the GEMM's SMs (a shared-memory request no GEMM SM can meet, the GEMM on 8-16 fewer SMs) was
  // slower still, 8-16 SMs cannot feed the link.
  push_tiles_kernel<<<static_cast<unsigned>(num_tiles * parts), 256, 0, stream>>>(
      static_cast<const unsigned char*>(c), pp, n_peers, pitch_bytes, m, n_bytes, tile_m, tile_n_bytes, tiles_m, tiles_n, group_m,
      first_tile, parts);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "push_tiles_kernel launch");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}

}  // namespace tb
