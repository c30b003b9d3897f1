// gemm_kernel instantiations of MMA kind 0 (f16), one CTA and CTA pair.
#define TB_GEMM_INSTANTIATE_KIND 0
#include "gemm_launch.cuh"
