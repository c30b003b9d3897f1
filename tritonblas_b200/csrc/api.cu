// C ABI of libtritonblas_b200.so: argument checking, tensor-map construction, kernel launches.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/tritonblas_b200.h"
#include "common_host.h"
#include "gemm_launch.cuh"
#include "selector.h"

namespace tb {

static thread_local char g_cuda_err[256] = "";
std::atomic<long long> g_launches{0};

int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: %s", what, cudaGetErrorString(e));
  return TB_ERR_CUDA;
}
int cu_fail(int code, const char* what) {
  snprintf(g_cuda_err, sizeof(g_cuda_err), "%s: CUresult %d", what, code);
  return TB_ERR_CUDA;
}

// ---------------------------------------------------------------- per-device state
struct DeviceState {
  bool ready = false;
  int num_sms = 0;
  int smem_optin = 0;
  int* status = nullptr;  // device address of g_status_word on this device
};
static DeviceState g_dev[64];
static std::mutex g_mu;  // guards g_dev and g_encode
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
// The word kernels write a failure code into. Part of the library image (one instance per GPU that loads it), so the
// library never calls an allocator; its device address is looked up once per device.
static __device__ int g_status_word;

// Makes `device` current for the lifetime of the object and puts the caller's device back on every exit path.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
    if (prev != device) {
      err = cudaSetDevice(device);
      switched = err == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (switched && prev >= 0) cudaSetDevice(prev);
  }
};

int device_state(int device, DeviceState** out) {
  if (device < 0 || device >= 64) return TB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& d = g_dev[device];
  if (!d.ready) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || device >= count) {
      cudaGetLastError();
      return TB_ERR_NO_DEVICE;
    }
    DeviceGuard guard(device);
    if (guard.err != cudaSuccess) return cuda_fail(guard.err, "cudaSetDevice");
    cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, device);
    cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    // In host code the symbol's name is not a device address: ask for it, with this device current.
    void* word = nullptr;
    if ((e = cudaGetSymbolAddress(&word, g_status_word)) != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(status)");
    d.status = static_cast<int*>(word);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
      if (e != cudaSuccess || fn == nullptr) return cuda_fail(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    d.ready = true;
  }
  *out = &d;
  return TB_OK;
}

int current_device_state(DeviceState** out, int* device) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return TB_ERR_NO_DEVICE;
  }
  if (device) *device = dev;
  return device_state(dev, out);
}

int* device_status_word(int device) {
  DeviceState* d = nullptr;
  if (device_state(device, &d) != TB_OK) return nullptr;
  return d->status;
}

static CUtensorMapDataType tmap_dtype(int dtype) {
  switch (dtype) {
    case TB_DTYPE_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case TB_DTYPE_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case TB_DTYPE_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    default: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  }
}

// 2-D row-major view [outer][inner] with `outer_stride_bytes` between rows; box = box_inner x box_outer elements.
int encode_2d(CUtensorMap* map, int dtype, const void* base, uint64_t inner, uint64_t outer, uint64_t outer_stride_bytes,
              uint32_t box_inner, uint32_t box_outer, int swizzle) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (outer_stride_bytes & 15) != 0) return TB_ERR_ALIGNMENT;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {outer_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, tmap_dtype(dtype), 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                     : (swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cu_fail(static_cast<int>(r), "cuTensorMapEncodeTiled");
  return TB_OK;
}

// MN-major operand [k][mn] (mn contiguous, `k_stride_bytes` between K rows) as a 3-D tensor [mn / atom][k][atom], atom =
// the elements of one 128-byte swizzle row: one box of `groups` atoms x box_k rows lands in shared memory atom after atom,
// the layout the MN-major matrix descriptors expect, with a single TMA instruction per operand and stage instead of one
// per atom. Needs mn to be a multiple of the atom; the driver may also refuse the stride order (the K stride, which is
// the larger one, comes first), in which case the caller keeps the 2-D map and one copy per atom.
int encode_mn3d(CUtensorMap* map, int dtype, const void* base, uint64_t mn, uint64_t k, uint64_t k_stride_bytes,
                uint32_t atom, uint32_t box_k, uint32_t groups, int swizzle) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (k_stride_bytes & 15) != 0) return TB_ERR_ALIGNMENT;
  if (mn % atom != 0 || groups == 0) return TB_ERR_UNSUPPORTED;
  cuuint64_t dims[3] = {atom, k, mn / atom};
  cuuint64_t strides[2] = {k_stride_bytes, 128};
  cuuint32_t box[3] = {atom, box_k, groups};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, tmap_dtype(dtype), 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TB_OK : TB_ERR_UNSUPPORTED;
}

// Scale-factor atoms as a 3-D tensor of 32-bit words: [row groups][K atoms][128 words]; box = one group x two atoms.
int encode_sf_atoms(CUtensorMap* map, const void* base, uint64_t k_atoms, uint64_t groups) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return TB_ERR_ALIGNMENT;
  cuuint64_t dims[3] = {128, k_atoms, groups};
  cuuint64_t strides[2] = {512, 512 * k_atoms};
  cuuint32_t box[3] = {128, 2, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return cu_fail(static_cast<int>(r), "cuTensorMapEncodeTiled(scale atoms)");
  return TB_OK;
}

static int esize_of(int dtype) {
  switch (dtype) {
    case TB_DTYPE_F16:
    case TB_DTYPE_BF16: return 2;
    case TB_DTYPE_F32: return 4;
    case TB_DTYPE_E4M3:
    case TB_DTYPE_E5M2:
    case TB_DTYPE_I8:
    case TB_DTYPE_U8: return 1;
    default: return 0;
  }
}

MachineModel machine_for(const DeviceState* d) {
  MachineModel hw;
  if (d != nullptr) {
    hw.num_sms = d->num_sms;
    hw.smem_optin = d->smem_optin;
  }
  // measurement knob, read once: TB_DISABLE_CTA_PAIR=1 keeps the model to single-CTA tiles
  static const bool no_pair = getenv("TB_DISABLE_CTA_PAIR") != nullptr && getenv("TB_DISABLE_CTA_PAIR")[0] == '1';
  if (no_pair) hw.allow_pair = false;
  return hw;
}

bool pdl_enabled() {
  static const bool on = getenv("TB_PDL") == nullptr || atoi(getenv("TB_PDL")) != 0;
  return on;
}

// ---------------------------------------------------------------- built-in stream-K scratch (tb_gemm_streamk_builtin)
// Flags (4 KB) followed by the fp32 partial tiles, in a device array that is part of the library image: every GPU that
// loads the library holds these bytes until the process exits. In host code the array's name only stands for the
// symbol; the address a kernel can use is asked for once per device, with that device current.
constexpr size_t kBuiltinFlagBytes = 4096;
constexpr size_t kBuiltinPartialBytes = 10u * 1024u * 1024u;
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinFlagBytes + kBuiltinPartialBytes];
static unsigned char* g_builtin_addr[64] = {};
static std::mutex g_builtin_mu;

static int builtin_scratch(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return TB_ERR_NO_DEVICE;
  }
  if (dev < 0 || dev >= 64) return TB_ERR_INVALID;
  std::lock_guard<std::mutex> lk(g_builtin_mu);
  if (g_builtin_addr[dev] == nullptr) {
    void* p = nullptr;
    if ((e = cudaGetSymbolAddress(&p, g_builtin_scratch)) != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(scratch)");
    g_builtin_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_builtin_addr[dev];
  return TB_OK;
}

int launch_push_tiles(const void* c, void* const* peers, int n_peers, long long pitch_bytes, int m, long long n_bytes, int tile_m,
                      int tile_n_bytes, int tiles_m, int tiles_n, int group_m, int first_tile, int num_tiles,
                      cudaStream_t stream);  // push_tiles.cu

// Tile grid of a dense data-parallel launch with this configuration: what the kernel enumerates and what a copy of
// the launch's tail tiles must enumerate the same way.
struct TileGrid {
  int pair, bn, halves, tiles_m, tiles_n, group_m;
};
static TileGrid tile_grid(const tb_gemm_args& a, const tb_config& cfg) {
  TileGrid g;
  g.pair = cfg.cta_pair == 2 ? 2 : 1;
  g.bn = cfg.block_n;
  g.halves = (cfg.n_halves == 2 && !a.streamk) ? 2 : 1;
  g.tiles_m = (a.m + 128 * g.pair - 1) / (128 * g.pair);
  g.tiles_n = (a.n + g.bn * g.halves - 1) / (g.bn * g.halves);
  g.group_m = cfg.group_m > 0 ? cfg.group_m : 8;
  return g;
}

int gemm_fp32_exact(const tb_gemm_args& a, cudaStream_t stream);                 // simt_gemm.cu
int gemm_generic_loader(const tb_gemm_args& a, const tb_config& cfg, cudaStream_t stream, int* status);  // unaligned operands

// `builtin`: the stream-K flags and partial tiles of this launch live in the library's own scratch array (the launch
// takes no workspace from the caller).
static int gemm_impl(const tb_gemm_args& a_in, const tb_config* user_cfg, cudaStream_t stream, bool grouped = false,
                     bool swapped = false, bool builtin = false) {
  const tb_gemm_args& a = a_in;
  if (a.m < 0 || a.n < 0 || a.k < 0) return TB_ERR_INVALID;
  if (grouped && (a.group_offsets == nullptr || a.num_groups <= 0 || a.num_groups > 4096 || a.streamk)) return TB_ERR_INVALID;
  if (a.m == 0 || a.n == 0) return TB_OK;
  if (a.c == nullptr || ((a.a == nullptr || a.b == nullptr) && a.k != 0)) return TB_ERR_INVALID;  // empty operands have no address
  if (a.a_dtype != a.b_dtype) return TB_ERR_UNSUPPORTED;
  const int es = esize_of(a.a_dtype);
  if (es == 0 || a.a_dtype == TB_DTYPE_U8) return TB_ERR_UNSUPPORTED;
  if (a.c_dtype != TB_DTYPE_F16 && a.c_dtype != TB_DTYPE_BF16 && a.c_dtype != TB_DTYPE_F32 && a.c_dtype != TB_DTYPE_E4M3 &&
      a.c_dtype != TB_DTYPE_I8)
    return TB_ERR_UNSUPPORTED;

  DeviceState* dev = nullptr;
  int device = 0;
  int rc = current_device_state(&dev, &device);
  if (rc != TB_OK) return rc;

  // An empty K range leaves the epilogue alone (zero, scaled, plus bias): the CUDA-core kernel's loop simply does not run.
  if ((a.a_dtype == TB_DTYPE_F32 && !a.allow_tf32) || a.k == 0) return grouped ? TB_ERR_UNSUPPORTED : gemm_fp32_exact(a, stream);

  // operand majors from strides
  int a_mn, b_mn;
  if (a.a_stride_k == 1 || a.k == 1) a_mn = 0;
  else if (a.a_stride_m == 1 || a.m == 1) a_mn = 1;
  else return TB_ERR_UNSUPPORTED;
  if (a.b_stride_k == 1 || a.k == 1) b_mn = 0;
  else if (a.b_stride_n == 1 || a.n == 1) b_mn = 1;
  else return TB_ERR_UNSUPPORTED;
  if (a.a_stride_k == 1 && a.a_stride_m == 1 && a.m > 1 && a.k > 1) return TB_ERR_INVALID;
  if (grouped && (a_mn || b_mn)) return TB_ERR_UNSUPPORTED;

  tb_config cfg;
  if (user_cfg != nullptr) {
    cfg = *user_cfg;
  } else {
    tb_problem pr = {};
    pr.m = a.m;  // grouped: tiles of all groups are pooled over the SMs, so the model sees the total row count
    pr.n = a.n; pr.k = a.k;
    pr.a_dtype = a.a_dtype; pr.b_dtype = a.b_dtype; pr.c_dtype = a.c_dtype;
    pr.a_mn_major = a_mn; pr.b_mn_major = b_mn;
    pr.streamk = a.streamk;
    pr.device = device;
    rc = select_config(pr, machine_for(dev), &cfg);
    if (rc != TB_OK) return rc;
  }
  if (cfg.swap_ab && !swapped && !grouped && a.epilogue_op == TB_EPILOGUE_NONE) {
    // C^T = B^T A^T: exchange the operands' roles and transpose the output view; the per-row and per-column epilogue
    // vectors trade places and the bias becomes a per-row vector.
    tb_gemm_args t = a;
    t.m = a.n; t.n = a.m;
    t.a = a.b; t.a_stride_m = a.b_stride_n; t.a_stride_k = a.b_stride_k;
    t.b = a.a; t.b_stride_k = a.a_stride_k; t.b_stride_n = a.a_stride_m;
    t.c_stride_m = a.c_stride_n; t.c_stride_n = a.c_stride_m;
    t.a_scale = a.b_scale; t.b_scale = a.a_scale;
    t.static_operands = ((a.static_operands & 1) << 1) | ((a.static_operands >> 1) & 1);
    tb_config c2 = cfg;
    c2.swap_ab = 0;
    rc = gemm_impl(t, &c2, stream, false, true, builtin);
    // Operands TMA cannot address go to the CUDA-core kernel in their original orientation (its bias is per column).
    if (rc == TB_ERR_ALIGNMENT) return gemm_generic_loader(a, cfg, stream, dev->status);
    return rc;
  }
  const bool glu = a.epilogue_op == TB_EPILOGUE_SWIGLU;
  if (a.epilogue_op != TB_EPILOGUE_NONE && !glu) return TB_ERR_INVALID;
  if (glu) {
    // gate and up columns side by side in every accumulator: whole tiles and the straight-line 16-bit drain only
    if (a.streamk || swapped || a_mn || b_mn || a.a_scale != nullptr || a.b_scale != nullptr || a.bias != nullptr ||
        a.num_c_copies != 0 || (a.c_dtype != TB_DTYPE_BF16 && a.c_dtype != TB_DTYPE_F16) ||
        a.a_dtype == TB_DTYPE_F32 || a.a_dtype == TB_DTYPE_I8)
      return TB_ERR_UNSUPPORTED;
    if (a.c_stride_n != 1 || ((a.c_stride_m * 2) & 15) != 0 || (reinterpret_cast<uintptr_t>(a.c) & 15) != 0)
      return TB_ERR_ALIGNMENT;
    if (cfg.swap_ab || (a.n % 128) != 0 || a.m <= 128) return TB_ERR_UNSUPPORTED;
    // CTA pair, 256-column accumulators (128 gate + 128 up columns), narrow tiles: the drain and its exponentials hide
    // behind the next tile's main loop
    cfg.cta_pair = 2;
    cfg.block_m = 256;
    cfg.block_n = 256;
    cfg.n_halves = 1;
  }
  const int pair = cfg.cta_pair == 2 ? 2 : 1;
  const int bn = cfg.block_n;
  const int mn_atom = 128 / es;
  if (bn < 32 || bn > 256 || (bn % 32) != 0 || cfg.block_m != 128 * pair) return TB_ERR_INVALID;
  if ((bn / pair) % 16 != 0) return TB_ERR_INVALID;
  if (b_mn && ((bn / pair) % mn_atom) != 0) return TB_ERR_INVALID;
  const int bk = 128 / es;
  // wide tiles (two accumulators sharing A) only for the data-parallel and grouped schedules: stream-K partials are per accumulator
  const int halves = (cfg.n_halves == 2 && !a.streamk) ? 2 : 1;
  int stages = cfg.stages;
  if (stages < 2) stages = 2;
  const int extra_smem = grouped ? 8 * (a.num_groups + 2) : 0;  // per-group tile prefix + copy of the row offsets
  while (stages > 2 && smem_bytes_for(bn, pair, stages, halves) + extra_smem > dev->smem_optin) --stages;
  const int smem_bytes = smem_bytes_for(bn, pair, stages, halves) + extra_smem;
  if (smem_bytes > dev->smem_optin) return TB_ERR_INVALID;

  GemmParams p = {};
  p.M = a.m; p.N = a.n; p.K = a.k;
  p.block_n = bn;
  p.n_halves = halves;
  p.k_per_stage = bk;
  p.num_k_blocks = (a.k + bk - 1) / bk;
  const TileGrid tgrid = tile_grid(a, cfg);
  p.tiles_m = tgrid.tiles_m;
  p.glu = glu ? 1 : 0;
  p.tiles_n = glu ? a.n / (bn / 2) : tgrid.tiles_n;
  p.group_m = tgrid.group_m;
  p.stages = stages;
  p.esize = es;
  p.a_mn = a_mn; p.b_mn = b_mn;
  int tc = 32;
  while (tc < 2 * bn) tc <<= 1;
  p.tmem_cols = static_cast<uint32_t>(tc);
  p.C = a.c; p.ldc_m = a.c_stride_m; p.ldc_n = a.c_stride_n; p.c_dtype = a.c_dtype;
  if (a.num_c_copies < 0 || a.num_c_copies > 7 || (a.num_c_copies > 0 && a.c_copies == nullptr)) return TB_ERR_INVALID;
  for (int x = 0; x < a.num_c_copies; ++x) p.c_extra[x] = a.c_copies[x];
  p.num_c_extra = a.num_c_copies;
  p.c_extra_tile_limit = a.c_copies_tile_limit > 0 ? a.c_copies_tile_limit : 0x7fffffff;
  {
    bool ok16 = (a.c_dtype == TB_DTYPE_BF16 || a.c_dtype == TB_DTYPE_F16) && a.c_stride_n == 1 && ((a.c_stride_m * 2) & 15) == 0 &&
                (reinterpret_cast<uintptr_t>(a.c) & 15) == 0;
    for (int x = 0; x < a.num_c_copies; ++x) ok16 = ok16 && (reinterpret_cast<uintptr_t>(a.c_copies[x]) & 15) == 0;
    p.staged_store = ok16 ? 1 : 0;
    p.staged_f32 = (a.c_dtype == TB_DTYPE_F32 && a.c_stride_n == 1 && ((a.c_stride_m * 4) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.c) & 15) == 0 && a.num_c_copies == 0)
                       ? 1
                       : 0;
  }
  p.a_scale = a.a_scale; p.b_scale = a.b_scale;
  p.bias = a.bias; p.bias_stride = a.bias_stride; p.bias_dtype = a.bias_dtype;
  p.bias_along_m = swapped ? 1 : 0;
  p.status = dev->status;
  // bound of every device-side wait: 2 s unless the caller asks for another one
  p.timeout_ns = a.wait_timeout_ms > 0 ? static_cast<unsigned long long>(a.wait_timeout_ms) * 1000000ull : 2000000000ull;
  if (grouped) {
    p.group_offsets = a.group_offsets;
    p.num_groups = a.num_groups;
  }
  const bool gather = a.a_gather_index != nullptr;
  if (gather) {
    // rows of A picked by index from another matrix: grouped launches of 16-bit K-contiguous operands that TMA can address
    if (!grouped || a_mn || es != 2 || a.a_stride_k != 1 || a.a_rows <= 0) return TB_ERR_UNSUPPORTED;
    p.a_gather = a.a_gather_index;
  }
  if (a.tile_counter != nullptr && !a.streamk) {
    if (reinterpret_cast<uintptr_t>(a.tile_counter) & 3) return TB_ERR_ALIGNMENT;
    p.tile_counter = static_cast<unsigned*>(a.tile_counter);
  }
  // An operand nothing in flight writes is requested before the wait for the previous kernel (single CTAs, static
  // schedules): the larger one per stage if both are.
  if (pair == 1 && !grouped && !gather && p.tile_counter == nullptr && pdl_enabled()) {
    if ((a.static_operands & 3) == 3) p.early_operand = bn * halves > 128 ? 2 : 1;
    else if (a.static_operands & 1) p.early_operand = 1;
    else if (a.static_operands & 2) p.early_operand = 2;
  }
  {
    p.debug_flags = a.debug_flags;
    // role cycle counters (148 x 16 words): the start of the workspace for data-parallel launches, its last 19 KB for
    // stream-K launches whose caller over-allocated by that much
    constexpr long long kDebugBytes = 148 * 16 * 8;
    p.debug_out = nullptr;
    if ((p.debug_flags & 2) && a.workspace != nullptr) {
      if (!a.streamk) p.debug_out = reinterpret_cast<long long*>(a.workspace);
      else if (a.workspace_bytes >= tb_gemm_workspace_bytes(&cfg, a.sk_grid) + kDebugBytes)
        p.debug_out = reinterpret_cast<long long*>(static_cast<char*>(a.workspace) + ((a.workspace_bytes - kDebugBytes) & ~7ll));
    }
    // Dense data-parallel launches: odd items walk K backwards (L2 reuse between consecutive tiles; +0.5-1 % sustained on
    // 8192^3). Not for grouped launches, where it measured 6 % slower on Zipf-sized groups.
    // Bit 3 of the debug flags turns it off for A/B measurements.
    p.k_serpentine = (!a.streamk && !grouped && !(p.debug_flags & 8)) ? 1 : 0;
  }

  // instruction descriptor: fp32 accumulate; operand formats; majors; N >> 3; M >> 4
  int kind;
  uint32_t fmt;
  switch (a.a_dtype) {
    case TB_DTYPE_F16: kind = 0; fmt = 0; break;
    case TB_DTYPE_BF16: kind = 0; fmt = 1; break;
    case TB_DTYPE_F32: kind = 1; fmt = 2; break;
    case TB_DTYPE_E4M3: kind = 2; fmt = 0; break;
    case TB_DTYPE_E5M2: kind = 2; fmt = 1; break;
    case TB_DTYPE_I8: kind = 4; fmt = 1; break;   // signed 8-bit
    default: return TB_ERR_UNSUPPORTED;
  }
  const uint32_t c_fmt = kind == 4 ? 2u : 1u;     // accumulator: int32 for the integer kind, fp32 otherwise
  p.idesc = (c_fmt << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_mn) << 15) | (static_cast<uint32_t>(b_mn) << 16) |
            (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>((128 * pair) >> 4) << 24);

  // schedule
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  const int max_programs = dev->num_sms / pair;
  int programs;
  if (a.streamk) {
    programs = a.sk_grid > 0 ? a.sk_grid : cfg.sk_grid;
    if (programs <= 0) programs = max_programs;
    // All programs of a stream-K launch must be resident at once: owners wait for peers.
    if (programs > max_programs) programs = max_programs;
    const long long total_iters = tiles * p.num_k_blocks;
    if (programs > total_iters) programs = static_cast<int>(total_iters);
    p.sk_tiles = static_cast<int>(tiles % programs);
    p.dp_tiles = static_cast<int>(tiles - p.sk_tiles);
    if (p.sk_tiles > 0 && builtin) {
      // one fp32 partial tile of 128 x block_n per CTA; launches without a split tile need none and are never refused
      const size_t need = static_cast<size_t>(programs) * pair * 128 * static_cast<size_t>(bn) * 4;
      if (need > kBuiltinPartialBytes || static_cast<size_t>(programs) * pair * 4 > kBuiltinFlagBytes) {
        snprintf(g_cuda_err, sizeof(g_cuda_err),
                 "built-in stream-K scratch holds %zu bytes of partial tiles, this launch needs %zu (%d programs x %d x 128 x %d "
                 "fp32); pass a smaller sk_grid or use tb_gemm with a caller workspace",
                 kBuiltinPartialBytes, need, programs, pair, bn);
        return TB_ERR_WORKSPACE;
      }
      unsigned char* scratch = nullptr;
      if ((rc = builtin_scratch(&scratch)) != TB_OK) return rc;
      p.flags = reinterpret_cast<unsigned*>(scratch);
      p.partials = reinterpret_cast<float*>(scratch + kBuiltinFlagBytes);
      p.epoch = 1;
      // The array keeps the previous call's contents: the flags must start at zero (partial tiles are written before
      // they are read).
      cudaError_t me = cudaMemsetAsync(scratch, 0, kBuiltinFlagBytes, stream);
      if (me != cudaSuccess) return cuda_fail(me, "cudaMemsetAsync(flags)");
    } else if (p.sk_tiles > 0) {
      const int64_t need = tb_gemm_workspace_bytes(&cfg, programs);
      if (a.workspace == nullptr || a.workspace_bytes < need) return TB_ERR_WORKSPACE;
      if (a.epoch == 0) return TB_ERR_INVALID;
      p.flags = reinterpret_cast<unsigned*>(a.workspace);
      p.partials = reinterpret_cast<float*>(reinterpret_cast<char*>(a.workspace) + 4096);
      p.epoch = a.epoch;
    }
  } else if (grouped) {
    programs = max_programs;  // the tile count depends on the device-side group sizes
    p.dp_tiles = 0;
    p.sk_tiles = 0;
  } else {
    programs = cfg.grid > 0 ? cfg.grid : max_programs;
    if (programs > max_programs) programs = max_programs;
    if (programs > tiles) programs = static_cast<int>(tiles);
    p.dp_tiles = static_cast<int>(tiles);
    p.sk_tiles = 0;
  }
  if (programs < 1) programs = 1;

  // tensor maps
  CUtensorMap ta, tbm;
  const void* A = a.a;
  const void* B = a.b;
  // swizzle: 1 = 128-byte rows of 16-byte chunks; 2 = 128-byte rows of 32-byte chunks (MN-major 32-bit operands)
  const int mn_swz = es == 4 ? 2 : 1;
  static const bool no_mn3d = getenv("TB_DISABLE_MN3D") != nullptr;  // measurement knob, read once
  if (gather) {
    // gather-mode copies take their rows from a map over the whole source matrix whose box is one row of a stage
    rc = encode_2d(&ta, a.a_dtype, A, a.k, a.a_rows, static_cast<uint64_t>(a.a_stride_m) * es, bk, 1, 1);
  } else if (!a_mn) {
    rc = encode_2d(&ta, a.a_dtype, A, a.k, a.m, static_cast<uint64_t>(a.a_stride_m) * es, bk, 128, 1);
  } else {
    // one 3-D copy per stage when the driver takes the map, else one 2-D copy per 128-byte atom
    if (!no_mn3d && encode_mn3d(&ta, a.a_dtype, A, a.m, a.k, static_cast<uint64_t>(a.a_stride_k) * es, mn_atom, bk,
                                128 / mn_atom, mn_swz) == TB_OK)
      p.a_mn3d = 1;
    else
      rc = encode_2d(&ta, a.a_dtype, A, a.m, a.k, static_cast<uint64_t>(a.a_stride_k) * es, mn_atom, bk, mn_swz);
  }
  if (rc == TB_OK) {
    const uint64_t b_rows = (grouped ? static_cast<uint64_t>(a.n) * a.num_groups : static_cast<uint64_t>(a.n)) * (glu ? 2 : 1);
    if (!b_mn) {
      rc = encode_2d(&tbm, a.b_dtype, B, a.k, b_rows, static_cast<uint64_t>(a.b_stride_n) * es, bk, bn / pair, 1);
    } else if (!no_mn3d && encode_mn3d(&tbm, a.b_dtype, B, a.n, a.k, static_cast<uint64_t>(a.b_stride_k) * es, mn_atom,
                                       bk, (bn / pair) / mn_atom, mn_swz) == TB_OK) {
      p.b_mn3d = 1;
    } else {
      rc = encode_2d(&tbm, a.b_dtype, B, a.n, a.k, static_cast<uint64_t>(a.b_stride_k) * es, mn_atom, bk, mn_swz);
    }
  }
  if (rc == TB_ERR_ALIGNMENT && !grouped && !swapped) return gemm_generic_loader(a, cfg, stream, dev->status);
  if (rc != TB_OK) return rc;

#define TB_LAUNCH(K, C) return launch_gemm<K, C>(ta, tbm, p, programs, smem_bytes, stream)
  if (pair == 1) {
    if (kind == 0) TB_LAUNCH(0, 1);
    if (kind == 1) TB_LAUNCH(1, 1);
    if (kind == 4) TB_LAUNCH(4, 1);
    TB_LAUNCH(2, 1);
  } else {
    if (kind == 0) TB_LAUNCH(0, 2);
    if (kind == 1) TB_LAUNCH(1, 2);
    if (kind == 4) TB_LAUNCH(4, 2);
    TB_LAUNCH(2, 2);
  }
#undef TB_LAUNCH
}

// ---------------------------------------------------------------- MXFP4 (block-scaled e2m1 x e2m1)
static int gemm_mxfp4_impl(const tb_mxfp4_args& a, cudaStream_t stream) {
  if (a.m < 0 || a.n < 0 || a.k < 0 || (a.k % 32) != 0) return TB_ERR_INVALID;
  if (a.m == 0 || a.n == 0) return TB_OK;
  if (a.k == 0) return TB_ERR_UNSUPPORTED;
  if (a.a == nullptr || a.b == nullptr || a.c == nullptr || a.a_scales == nullptr || a.b_scales == nullptr) return TB_ERR_INVALID;
  if (a.scales_in_atoms != 1) return TB_ERR_UNSUPPORTED;  // row-major scales are re-arranged by tb_mxfp4_scales_to_atoms first
  if (a.c_dtype != TB_DTYPE_F16 && a.c_dtype != TB_DTYPE_BF16 && a.c_dtype != TB_DTYPE_F32) return TB_ERR_UNSUPPORTED;
  DeviceState* dev = nullptr;
  int device = 0;
  int rc = current_device_state(&dev, &device);
  if (rc != TB_OK) return rc;

  tb_config cfg;
  tb_problem pr = {};
  pr.m = a.m; pr.n = a.n; pr.k = a.k;
  pr.a_dtype = pr.b_dtype = TB_DTYPE_F4; pr.c_dtype = a.c_dtype;
  pr.mx_block_size = 32;
  pr.device = device;
  rc = select_config(pr, machine_for(dev), &cfg);
  if (rc != TB_OK) return rc;
  if (a.block_n > 0) cfg.block_n = a.block_n;
  if (a.cta_pair > 0) cfg.cta_pair = a.cta_pair;
  if (a.group_m > 0) cfg.group_m = a.group_m;
  const int pair = cfg.cta_pair == 2 ? 2 : 1;
  const int bn = cfg.block_n;
  const int groups = kSfGroupsB;  // 128-row scale groups staged per tile
  // Widths are multiples of 64: the MMA reads B's scale factors starting at an even TMEM column (64 rows apart).
  if (bn < 64 || bn > 192 || (bn % 64) != 0) return TB_ERR_INVALID;
  const int kbytes = a.k / 2;
  const int stage_bytes = (128 * 128 + (bn / pair) * 128 + (2 + 2 * groups) * 512 + 1023) & ~1023;
  int stages = (dev->smem_optin - 2048 - kEpiStageBytes) / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages < 2) return TB_ERR_INVALID;
  const int smem_bytes = stages * stage_bytes + kEpiStageBytes + (2 * stages + 16) * 8 + 64 + 1024;

  GemmParams p = {};
  p.M = a.m; p.N = a.n; p.K = a.k;
  p.block_n = bn;
  p.n_halves = 1;
  p.k_per_stage = 128;  // bytes of packed K per stage (256 elements)
  p.num_k_blocks = (kbytes + 127) / 128;
  p.tiles_m = (a.m + 128 * pair - 1) / (128 * pair);
  p.tiles_n = (a.n + bn - 1) / bn;
  p.group_m = cfg.group_m > 0 ? cfg.group_m : 8;
  p.stages = stages;
  p.esize = 1;
  p.a_mn = 0; p.b_mn = 0;
  int tc = 32;
  while (tc < 2 * bn + 8 + 8 * groups) tc <<= 1;
  p.tmem_cols = static_cast<uint32_t>(tc);
  p.C = a.c; p.ldc_m = a.c_stride_m; p.ldc_n = a.c_stride_n; p.c_dtype = a.c_dtype;
  p.staged_store = ((a.c_dtype == TB_DTYPE_BF16 || a.c_dtype == TB_DTYPE_F16) && a.c_stride_n == 1 &&
                    ((a.c_stride_m * 2) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.c) & 15) == 0) ? 1 : 0;
  p.status = dev->status;
  p.timeout_ns = 2000000000ull;
  // e2m1 operands (format 1), ue8m0 scales (bit 23), K-major, N >> 3, M >> 4; scale-factor ids are set per MMA
  p.idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) | (1u << 23) |
            (static_cast<uint32_t>((128 * pair) >> 4) << 24);
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  int programs = dev->num_sms / pair;
  if (programs > tiles) programs = static_cast<int>(tiles);
  if (programs < 1) programs = 1;
  p.dp_tiles = static_cast<int>(tiles);
  p.sk_tiles = 0;

  CUtensorMap ta, tbm;
  rc = encode_2d(&ta, TB_DTYPE_U8, a.a, kbytes, a.m, static_cast<uint64_t>(a.a_row_stride), 128, 128, 1);
  if (rc == TB_OK) rc = encode_2d(&tbm, TB_DTYPE_U8, a.b, kbytes, a.n, static_cast<uint64_t>(a.b_row_stride), 128, bn / pair, 1);
  CUtensorMap tsfa, tsfb;
  const uint64_t k_atoms = (static_cast<uint64_t>(a.k) + 127) / 128;
  if (rc == TB_OK) rc = encode_sf_atoms(&tsfa, a.a_scales, k_atoms, (static_cast<uint64_t>(a.m) + 127) / 128);
  if (rc == TB_OK) rc = encode_sf_atoms(&tsfb, a.b_scales, k_atoms, (static_cast<uint64_t>(a.n) + 127) / 128);
  if (rc != TB_OK) return rc;
  if (pair == 1) return launch_gemm<3, 1>(ta, tbm, p, programs, smem_bytes, stream, &tsfa, &tsfb);
  return launch_gemm<3, 2>(ta, tbm, p, programs, smem_bytes, stream, &tsfa, &tsfb);
}

// Stream-K launch on the built-in scratch: the regular launch path with the library's own flags and partial tiles.
static int gemm_streamk_builtin_impl(const tb_gemm_args& in, const tb_config* user_cfg, cudaStream_t stream,
                                     int32_t* prev_status) {
  if (in.m <= 0 || in.n <= 0 || in.k <= 0) return TB_ERR_INVALID;
  if (in.a == nullptr || in.b == nullptr || in.c == nullptr) return TB_ERR_INVALID;
  // what the regular entry point would route elsewhere or fan out is not offered here
  if (in.epilogue_op != TB_EPILOGUE_NONE || in.group_offsets != nullptr || in.num_groups != 0 || in.num_c_copies != 0)
    return TB_ERR_UNSUPPORTED;
  DeviceState* dev = nullptr;
  int device = 0;
  int rc = current_device_state(&dev, &device);
  if (rc != TB_OK) return rc;
  if (prev_status != nullptr) {
    // Outcome of the work enqueued before this call (waits for `stream`), then cleared.
    int v = 0;
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess) e = cudaMemcpy(&v, dev->status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && v != 0) e = cudaMemset(dev->status, 0, sizeof(int));
    if (e != cudaSuccess) return cuda_fail(e, "tb_gemm_streamk_builtin(status read)");
    *prev_status = v;
  }
  tb_gemm_args a = in;
  a.streamk = 1;
  a.workspace = nullptr;
  a.workspace_bytes = 0;
  a.epoch = 0;
  a.tile_counter = nullptr;
  return gemm_impl(a, user_cfg, stream, false, false, true);
}

}  // namespace tb

// ====================================================================== exported C ABI
extern "C" {

int tb_select(const tb_problem* p, tb_config* cfg) {
  if (p == nullptr || cfg == nullptr) return TB_ERR_INVALID;
  tb::DeviceState* dev = nullptr;
  // Without a usable device the model falls back to the B200 constants, so the selector also works on a CPU host.
  if (tb::device_state(p->device, &dev) != TB_OK) dev = nullptr;
  return tb::select_config(*p, tb::machine_for(dev), cfg);
}

int64_t tb_gemm_workspace_bytes(const tb_config* cfg, int32_t sk_grid_override) {
  if (cfg == nullptr) return 0;
  const int64_t programs = sk_grid_override > 0 ? sk_grid_override : (cfg->sk_grid > 0 ? cfg->sk_grid : cfg->num_sms);
  const int64_t pair = cfg->cta_pair == 2 ? 2 : 1;
  // 4 KB of flags, then one fp32 partial tile of 128 x block_n per CTA
  return 4096 + programs * pair * 128 * static_cast<int64_t>(cfg->block_n) * 4;
}

int tb_gemm(const tb_gemm_args* args, const tb_config* cfg, void* stream) {
  if (args == nullptr) return TB_ERR_INVALID;
  return tb::gemm_impl(*args, cfg, static_cast<cudaStream_t>(stream));
}

int tb_gemm_tile_count(const tb_gemm_args* args, const tb_config* cfg) {
  if (args == nullptr || cfg == nullptr || args->m <= 0 || args->n <= 0 || cfg->block_n <= 0) return 0;
  const tb::TileGrid g = tb::tile_grid(*args, *cfg);
  return g.tiles_m * g.tiles_n;
}

int tb_push_c_tiles(const tb_gemm_args* args, const tb_config* cfg, int32_t first_tile, void* stream) {
  if (args == nullptr || cfg == nullptr || args->c == nullptr || first_tile < 0) return TB_ERR_INVALID;
  if (args->num_c_copies < 0 || args->num_c_copies > 7 || (args->num_c_copies > 0 && args->c_copies == nullptr)) return TB_ERR_INVALID;
  if (cfg->swap_ab || args->streamk || args->group_offsets != nullptr || args->epilogue_op != TB_EPILOGUE_NONE) return TB_ERR_UNSUPPORTED;
  const int es = tb::esize_of(args->c_dtype);
  if (es == 0 || args->c_stride_n != 1) return TB_ERR_UNSUPPORTED;
  const long long pitch = args->c_stride_m * es, n_bytes = static_cast<long long>(args->n) * es;
  if ((pitch & 15) || (n_bytes & 15) || (reinterpret_cast<uintptr_t>(args->c) & 15)) return TB_ERR_ALIGNMENT;
  for (int x = 0; x < args->num_c_copies; ++x)
    if (reinterpret_cast<uintptr_t>(args->c_copies[x]) & 15) return TB_ERR_ALIGNMENT;
  const tb::TileGrid g = tb::tile_grid(*args, *cfg);
  const int tiles = g.tiles_m * g.tiles_n;
  if (first_tile >= tiles) return TB_OK;
  return tb::launch_push_tiles(args->c, args->c_copies, args->num_c_copies, pitch, args->m, n_bytes, 128 * g.pair,
                               g.bn * g.halves * es, g.tiles_m, g.tiles_n, g.group_m, first_tile, tiles - first_tile,
                               static_cast<cudaStream_t>(stream));
}

int tb_gemm_streamk_builtin(const tb_gemm_args* args, const tb_config* cfg, void* stream, int32_t* prev_status) {
  if (args == nullptr) return TB_ERR_INVALID;
  return tb::gemm_streamk_builtin_impl(*args, cfg, static_cast<cudaStream_t>(stream), prev_status);
}

int tb_grouped_gemm(const tb_gemm_args* args, const tb_config* cfg, void* stream) {
  if (args == nullptr) return TB_ERR_INVALID;
  return tb::gemm_impl(*args, cfg, static_cast<cudaStream_t>(stream), true);
}

int tb_gemm_mxfp4(const tb_mxfp4_args* args, void* stream) {
  if (args == nullptr) return TB_ERR_INVALID;
  return tb::gemm_mxfp4_impl(*args, static_cast<cudaStream_t>(stream));
}

int tb_device_status(int32_t device, int32_t* status_out) {
  tb::DeviceState* d = nullptr;
  int rc = tb::device_state(device, &d);
  if (rc != TB_OK) return rc;
  tb::DeviceGuard guard(device);
  if (guard.err != cudaSuccess) return tb::cuda_fail(guard.err, "cudaSetDevice");
  int v = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && v != 0) e = cudaMemset(d->status, 0, sizeof(int));
  if (e != cudaSuccess) return tb::cuda_fail(e, "tb_device_status");
  if (status_out) *status_out = v;
  return TB_OK;
}

int tb_device_info(int32_t device, int32_t* num_sms, int32_t* smem_optin_bytes) {
  tb::DeviceState* d = nullptr;
  int rc = tb::device_state(device, &d);
  if (rc != TB_OK) return rc;
  if (num_sms) *num_sms = d->num_sms;
  if (smem_optin_bytes) *smem_optin_bytes = d->smem_optin;
  return TB_OK;
}

const char* tb_status_string(int code) {
  switch (code) {
    case TB_OK: return "ok";
    case TB_ERR_INVALID: return "invalid argument";
    case TB_ERR_UNSUPPORTED: return "unsupported dtype, layout or shape";
    case TB_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
    case TB_ERR_WORKSPACE: return "stream-K workspace missing or too small";
    case TB_ERR_CUDA: return "CUDA call failed";
    case TB_ERR_NO_DEVICE: return "no usable CUDA device";
    case tb::TB_DEV_TIMEOUT_SMEM_EMPTY: return "device: producer timed out waiting for a free shared-memory stage";
    case tb::TB_DEV_TIMEOUT_SMEM_FULL: return "device: MMA issuer timed out waiting for a TMA-filled stage";
    case tb::TB_DEV_TIMEOUT_TMEM_EMPTY: return "device: MMA issuer timed out waiting for a drained accumulator";
    case tb::TB_DEV_TIMEOUT_TMEM_FULL: return "device: epilogue timed out waiting for an accumulator";
    case tb::TB_DEV_TIMEOUT_PEER_FLAG: return "device: stream-K owner timed out waiting for a peer's partial tile";
    case tb::TB_DEV_TIMEOUT_SCALE: return "device: timed out waiting for block scales";
    case tb::TB_DEV_TIMEOUT_STORE: return "device: timed out publishing a partial tile";
    case tb::TB_DEV_TIMEOUT_TILE_QUEUE: return "device: a role timed out waiting for the next tile of the dynamic schedule";
    default: return "unknown status";
  }
}

const char* tb_last_cuda_error(void) { return tb::g_cuda_err; }

int64_t tb_launch_count(void) { return tb::g_launches.load(); }

}  // extern "C"
