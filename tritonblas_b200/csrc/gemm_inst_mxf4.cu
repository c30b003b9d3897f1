// gemm_kernel instantiations of MMA kind 3 (mxf4), one CTA and CTA pair.
#define TB_GEMM_INSTANTIATE_KIND 3
#include "gemm_launch.cuh"
