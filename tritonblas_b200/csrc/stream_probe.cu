// Diagnostic: the rate at which the SMs can pull a K-major matrix out of HBM with the GEMM's own access pattern, and
// nothing else going on: one CTA per SM, one thread of it keeps `stages` TMA boxes of box_rows rows x 128 bytes in flight
// (row blocks dealt round-robin to the CTAs, K walked in 128-byte steps), and the data is dropped. This is the ceiling of
// the streaming phase of the decode-shaped GEMMs (few rows of activations against a wide weight matrix).
#include <cstdint>

#include "common_host.h"
#include "ptx.cuh"

namespace tb {

constexpr int kProbeSmemBytes = 200 * 1024;  // more than half an SM's shared memory: one CTA per SM

__global__ void __launch_bounds__(32, 1)
tma_stream_probe_kernel(const __grid_constant__ CUtensorMap tmap, int row_blocks, int kblocks, int stages, int box_rows,
                        int inner_step, int* status, unsigned long long timeout_ns) {
  extern __shared__ uint8_t probe_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(probe_smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int box_bytes = box_rows * 128;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(stages) * box_bytes);
  __shared__ int abort_flag;
  if (threadIdx.x != 0) return;
  abort_flag = 0;
  const WaitCtx wctx{&abort_flag, status, timeout_ns};
  for (int s = 0; s < stages; ++s) mbar_init(&full[s], 1);
  mbar_fence_init();
  long long total = 0;
  for (int rb = blockIdx.x; rb < row_blocks; rb += gridDim.x) total += kblocks;
  long long issued = 0, done = 0;
  int rb_i = blockIdx.x, kb_i = 0, s_issue = 0, s_wait = 0;
  uint32_t ph = 0;
  while (done < total) {
    while (issued < total && issued - done < stages) {
      mbar_arrive_expect_tx(&full[s_issue], static_cast<uint32_t>(box_bytes));
      tma_load_2d(smem + static_cast<size_t>(s_issue) * box_bytes, &tmap, &full[s_issue], kb_i * inner_step, rb_i * box_rows);
      if (++kb_i == kblocks) {
        kb_i = 0;
        rb_i += gridDim.x;
      }
      if (++s_issue == stages) s_issue = 0;
      ++issued;
    }
    // a wait that gives up leaves the failure code in the status word; the copies still in flight land in this CTA's
    // shared memory, which stays allocated until the loop below has seen them or given up on them too
    if (!mbar_wait(&full[s_wait], ph, wctx, TB_DEV_TIMEOUT_SMEM_FULL)) break;
    if (++s_wait == stages) {
      s_wait = 0;
      ph ^= 1;
    }
    ++done;
  }
  if (done < total) {
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
  }
}

}  // namespace tb

extern "C" int tb_tma_stream_probe(const void* base, int64_t rows, int64_t row_bytes, int64_t pitch_bytes, int32_t stages,
                                   int32_t box_rows, int32_t programs, void* stream) {
  if (base == nullptr || rows <= 0 || row_bytes < 128 || stages < 1 || programs < 1) return TB_ERR_INVALID;
  if (box_rows < 8 || box_rows > 256 || (box_rows & 7)) return TB_ERR_INVALID;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15) || (row_bytes & 127) || row_bytes > pitch_bytes) return TB_ERR_ALIGNMENT;
  if (static_cast<int64_t>(stages) * box_rows * 128 + 2048 + 8 * stages > tb::kProbeSmemBytes) return TB_ERR_INVALID;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return tb::cuda_fail(e, "cudaGetDevice");
  int* status = tb::device_status_word(device);
  if (status == nullptr) return TB_ERR_CUDA;
  CUtensorMap tm;
  // the matrix as 16-bit elements: 64 of them per 128-byte step
  int rc = tb::encode_2d(&tm, TB_DTYPE_BF16, base, static_cast<uint64_t>(row_bytes / 2), static_cast<uint64_t>(rows),
                         static_cast<uint64_t>(pitch_bytes), 64, static_cast<uint32_t>(box_rows), 1);
  if (rc != TB_OK) return rc;
  e = cudaFuncSetAttribute(tb::tma_stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, tb::kProbeSmemBytes);
  if (e != cudaSuccess) return tb::cuda_fail(e, "cudaFuncSetAttribute(probe)");
  const int row_blocks = static_cast<int>(rows / box_rows);  // whole boxes only
  tb::tma_stream_probe_kernel<<<static_cast<unsigned>(programs), 32, tb::kProbeSmemBytes, static_cast<cudaStream_t>(stream)>>>(
      tm, row_blocks, static_cast<int>(row_bytes / 128), stages, box_rows, 64, status, 2000000000ull);
  e = cudaGetLastError();
  if (e != cudaSuccess) return tb::cuda_fail(e, "tma_stream_probe_kernel launch");
  tb::g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}
