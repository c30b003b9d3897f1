// Launch wrapper of gemm_kernel<KIND, CTAS>. The kernel instantiations are the expensive part of the build, so each MMA
// kind is compiled in a translation unit of its own (gemm_inst_*.cu define TB_GEMM_INSTANTIATE_KIND and include this
// file); every other file only sees the declaration.
#pragma once
#include <mutex>

#include "common_host.h"
#include "gemm_sm100.cuh"

namespace tb {

// Enqueue one launch of gemm_kernel<KIND, CTAS> with `programs` programs (CTAs, or CTA pairs when CTAS == 2).
// tsfa / tsfb: scale-factor tensor maps of the block-scaled kind, null otherwise.
template <int KIND, int CTAS>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb_, const GemmParams& p, int programs, int smem_bytes,
                cudaStream_t stream, const CUtensorMap* tsfa = nullptr, const CUtensorMap* tsfb = nullptr);

// Programmatic dependent launch is on unless TB_PDL=0 was in the environment when the library made its first launch.
bool pdl_enabled();

#ifdef TB_GEMM_INSTANTIATE_KIND
template <int KIND, int CTAS>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb_, const GemmParams& p, int programs, int smem_bytes,
                cudaStream_t stream, const CUtensorMap* tsfa, const CUtensorMap* tsfb) {
  auto kernel = gemm_kernel<KIND, CTAS, false>;
  int variant = 0;
  // The instantiations with per-role cycle counters (measurement runs) and with a row-gathering A loader (grouped
  // launches whose rows are picked from another matrix by index) exist for 16-bit operands only.
  if constexpr (KIND == 0) {
    if (p.a_gather != nullptr) {
      kernel = gemm_kernel<KIND, CTAS, false, true>;
      variant = 2;
    } else if ((p.debug_flags & 2) && p.debug_out != nullptr) {
      kernel = gemm_kernel<KIND, CTAS, true>;
      variant = 1;
    }
  } else if (p.a_gather != nullptr) {
    return TB_ERR_UNSUPPORTED;
  }
  // The opt-in shared-memory size is set once per kernel instantiation and device (and again if a launch needs more).
  static int configured[3][64] = {};
  static std::mutex configured_mu;
  int dev_index = 0;
  cudaGetDevice(&dev_index);
  cudaError_t e = cudaSuccess;
  {
    std::lock_guard<std::mutex> lk(configured_mu);
    int& have = configured[variant][dev_index & 63];
    if (smem_bytes > have) {
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
      if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(smem)");
      have = smem_bytes;
    }
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(static_cast<unsigned>(programs * CTAS), 1, 1);
  lc.blockDim = dim3(gemm_threads<KIND>(), 1, 1);
  lc.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  // Programmatic dependent launch: this kernel's CTAs may be scheduled, and run their shared-memory prologue, while the
  // previous kernel of the stream drains; they wait for it (griddepcontrol.wait) before they touch global memory.
  // Measured: 2 us off an 85 us decode GEMM, 5 us off back-to-back small GEMMs.
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    lc.numAttrs = 2;
  }
  // Kinds without block scales never touch the scale maps; they get copies of the operand maps as placeholders.
  e = cudaLaunchKernelEx(&lc, kernel, ta, tb_, tsfa != nullptr ? *tsfa : ta, tsfb != nullptr ? *tsfb : tb_, p);
  if (e != cudaSuccess) return cuda_fail(e, "cudaLaunchKernelEx(gemm)");
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return TB_OK;
}
template int launch_gemm<TB_GEMM_INSTANTIATE_KIND, 1>(const CUtensorMap&, const CUtensorMap&, const GemmParams&, int, int,
                                                      cudaStream_t, const CUtensorMap*, const CUtensorMap*);
template int launch_gemm<TB_GEMM_INSTANTIATE_KIND, 2>(const CUtensorMap&, const CUtensorMap&, const GemmParams&, int, int,
                                                      cudaStream_t, const CUtensorMap*, const CUtensorMap*);
#endif

}  // namespace tb
