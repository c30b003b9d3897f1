// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (bulk tensor copies), tcgen05 (MMA, TMEM).
// Every wait in here is bounded: after a time limit it records a status code and tells the caller to unwind.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// Status codes written by kernels into the device status word (0 = ok).
enum : int {
  TB_DEV_OK = 0,
  TB_DEV_TIMEOUT_SMEM_EMPTY = 101,   // producer waited for a free shared-memory stage
  TB_DEV_TIMEOUT_SMEM_FULL = 102,    // MMA issuer waited for a TMA-filled stage
  TB_DEV_TIMEOUT_TMEM_EMPTY = 103,   // MMA issuer waited for the epilogue to drain an accumulator
  TB_DEV_TIMEOUT_TMEM_FULL = 104,    // epilogue waited for an accumulator
  TB_DEV_TIMEOUT_PEER_FLAG = 105,    // stream-K tile owner waited for a peer's partial tile
  TB_DEV_TIMEOUT_SCALE = 106,        // block-scale copy wait
  TB_DEV_TIMEOUT_STORE = 107,
  TB_DEV_TIMEOUT_TILE_QUEUE = 108,   // a role waited for the next tile index of the dynamic schedule
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Map a shared::cta address of this CTA to the shared::cluster address of the same offset in CTA `rank`.
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Programmatic dependent launch: let the next kernel of the stream start being scheduled, and wait for the previous one
// to have completed (both are no-ops for a kernel launched without the attribute).
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrive on a barrier that lives in another CTA of the cluster (address from mapa_cluster).
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Store to the shared memory of another CTA of the cluster (address from mapa_cluster).
__device__ __forceinline__ void st_shared_cluster_u32(uint32_t cluster_addr, uint32_t v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
// try_wait that also acquires writes made by other CTAs of the cluster before their (cluster-scope) arrive.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Shared by all waits of one CTA: where to record a failure and how long to wait.
struct WaitCtx {
  volatile int* abort_flag;   // in shared memory; set by the first wait that gives up
  int* status;                // in global memory; first failure code wins
  unsigned long long timeout_ns;
};

// Bounded wait on an mbarrier phase. Returns false if the CTA has to unwind (time limit hit here or elsewhere).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFF) == 0) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        *w.abort_flag = 1;
        atomicCAS(w.status, 0, code);
        return false;
      }
    }
  }
}

// The same bounded wait with a cluster-scope acquire (data written by the other CTA of a pair before its arrive).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 0xFF) == 0) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        *w.abort_flag = 1;
        atomicCAS(w.status, 0, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint32_t sm_id() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}

// One lane of a converged warp (all 32 lanes must call this together).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// Warp-collective bounded wait: every lane of a converged warp calls it and every lane gets the same answer, so the
// caller's control flow stays warp-uniform (which lets the compiler keep descriptors in uniform registers).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, const WaitCtx& w, int code) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  bool ok = true;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, w, code);
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  // The phase cannot advance again before this warp acts, so each lane's own acquiring test succeeds at once.
  if (ok) {
    for (int i = 0; i < 1024 && !mbar_try_wait(bar, parity); ++i) {
    }
  }
  return ok;
}

// Bounded wait until *flag == want (acquire at gpu scope). Used for stream-K partial-tile hand-off.
__device__ __forceinline__ bool flag_wait(const unsigned* flag, unsigned want, const WaitCtx& w, int code) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
  if (v == want) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == want) return true;
    if ((++spins & 0x3F) == 0) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() - t0 > w.timeout_ns) {
        *w.abort_flag = 1;
        atomicCAS(w.status, 0, code);
        return false;
      }
    }
    __nanosleep(spins < 8 ? 64 : 256);  // short waits stay short, long ones poll L2 four times less often
  }
}
__device__ __forceinline__ void flag_release(unsigned* flag, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(v) : "memory");
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 2-D tile load global -> shared, completion counted in bytes on `bar` (a barrier of this CTA).
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Same, issued inside a CTA pair: `bar_cluster_addr` may name a barrier of the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Gather-mode 2-D load: four rows (y0..y3, any order, out-of-range rows read as the fill value) of a tensor map whose box
// is ONE row of `x`-extent; they land as four consecutive rows at smem_dst and complete 4 x box bytes on the barrier.
__device__ __forceinline__ void tma_gather4_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int x, int y0, int y1,
                                               int y2, int y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
      : "memory");
}
__device__ __forceinline__ void tma_gather4_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int x,
                                                    int y0, int y1, int y2, int y3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.cta_group::2 [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::
          "r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
      : "memory");
}
// 2-D tile store shared -> global (bulk group completion).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* tmap, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(tmap),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy (TMA store, tcgen05 reads).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05 / TMEM
template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols)
                 : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// MMA kinds: 0 = f16/bf16 operands, 1 = tf32, 2 = 8-bit floats (e4m3/e5m2), 4 = signed 8-bit integers (int32 accumulate).
template <int KIND, int CTAS>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
#define TB_UMMA(G, K)                                                                            \
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"                                 \
               "tcgen05.mma.cta_group::" G ".kind::" K " [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d), \
               "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)                               \
               : "memory")
  if constexpr (CTAS == 1) {
    if constexpr (KIND == 0) TB_UMMA("1", "f16");
    else if constexpr (KIND == 1) TB_UMMA("1", "tf32");
    else if constexpr (KIND == 4) TB_UMMA("1", "i8");
    else TB_UMMA("1", "f8f6f4");
  } else {
    if constexpr (KIND == 0) TB_UMMA("2", "f16");
    else if constexpr (KIND == 1) TB_UMMA("2", "tf32");
    else if constexpr (KIND == 4) TB_UMMA("2", "i8");
    else TB_UMMA("2", "f8f6f4");
  }
#undef TB_UMMA
}

// Block-scaled MXFP4 MMA (e2m1 operands, ue8m0 scale per 32 K elements), scales already in TMEM.
template <int CTAS>
__device__ __forceinline__ void umma_mxf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
  if constexpr (CTAS == 1)
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
  else
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n\t}" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb), "r"(accumulate)
        : "memory");
}

// Shared memory -> TMEM copy of 32 lanes x 128 bits, replicated to all four lane quadrants (scale factors).
template <int CTAS>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  if constexpr (CTAS == 1)
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
  else
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

// mbarrier arrive once all tcgen05 operations issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// CTA-pair form: arrive on the barrier at the same offset in every CTA named by `cta_mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(cta_mask)
               : "memory");
}

// TMEM -> registers: this warp's 32 lanes x 32 consecutive 32-bit columns (thread i gets lane i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]),
        "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]),
        "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, with the loaded registers passed through it: a load issued ahead of its use then has a true
// dependency on the wait, so no use of the registers can be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                 "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                 "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose base is 1024-byte aligned.
//   K-major : rows of 128 bytes (one row per M/N index), 8-row groups 1024 bytes apart (stride_bytes = 1024).
//   MN-major: 64x8-element-class atoms; lead_bytes = distance between atoms along M/N, stride_bytes = between 8-row K groups.
//   layout_type: 2 = 128-byte swizzle of 16-byte chunks (8-row pattern); 1 = 128-byte swizzle of 32-byte chunks
//   (4-row pattern), the only swizzled form the tensor core accepts for MN-major 32-bit operands.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lead_bytes, uint32_t stride_bytes,
                                                   uint32_t layout_type = 2) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lead_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;  // descriptor version for this architecture
  d |= static_cast<uint64_t>(layout_type) << 61;
  return d;
}
// Descriptor for unswizzled 8x16-byte core matrices (used for scale-factor copies into TMEM).
__device__ __forceinline__ uint64_t make_smem_desc_noswizzle(uint32_t smem_addr, uint32_t lead_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lead_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= 1ull << 46;
  return d;
}

}  // namespace tb
