// Host-side declarations shared by the translation units of libtritonblas_b200.so.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/tritonblas_b200.h"

namespace tb {

extern std::atomic<long long> g_launches;

int cuda_fail(cudaError_t e, const char* what);
int cu_fail(int code, const char* what);

// Device word that kernels write a failure code into (allocated once per device by the library).
int* device_status_word(int device);

// 2-D row-major tensor map [outer][inner]; box = box_inner x box_outer elements.
int encode_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer, uint64_t outer_stride_bytes,
              uint32_t box_inner, uint32_t box_outer, int swizzle);  // swizzle: 0 none, 1 128B, 2 128B with 32-byte chunks

}  // namespace tb
