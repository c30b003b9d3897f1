// gemm_kernel instantiations of MMA kind 4 (i8), one CTA and CTA pair.
#define TB_GEMM_INSTANTIATE_KIND 4
#include "gemm_launch.cuh"
