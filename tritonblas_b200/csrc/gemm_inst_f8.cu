// gemm_kernel instantiations of MMA kind 2 (f8), one CTA and CTA pair.
#define TB_GEMM_INSTANTIATE_KIND 2
#include "gemm_launch.cuh"
