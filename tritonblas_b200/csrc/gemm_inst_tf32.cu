// gemm_kernel instantiations of MMA kind 1 (tf32), one CTA and CTA pair.
#define TB_GEMM_INSTANTIATE_KIND 1
#include "gemm_launch.cuh"
