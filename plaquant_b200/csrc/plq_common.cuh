// Shared host/device helpers for libplq_b200: status handling, argument checks and the
// sm_100a PTX wrappers (mbarrier, bulk/TMA copies, tcgen05) used by the kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/plq.h"

namespace plq {

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return PLQ_ERR_CUDA;
}

#define PLQ_CUDA_TRY(expr)                                  \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) return ::plq::cuda_fail(_e);     \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 0 when the current device is compute capability 10.x (cached per device).
int device_check();
int sm_count();

// Byte offset of scale (row r, scale index kb) inside a PLQ_SF_TILED buffer with
// `chunks_k` = ceil(n_sf / 4) chunks per 128-row group.
__host__ __device__ inline int64_t sf_tiled_offset(int64_t r, int64_t kb, int64_t chunks_k) {
  return ((r >> 7) * chunks_k + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}

// ---------------------------------------------------------------------------------------
// Device side: PTX wrappers.  Every wait is bounded in wall-clock time.
// ---------------------------------------------------------------------------------------
#ifdef __CUDACC__

constexpr long long kWaitLimitCycles = 4000000000ll;   // ~2 s of SM clock per wait, then give up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
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

// Waits for the phase with the given parity to complete.  Returns false when `*abort` was
// set by another role of the CTA or when the time limit ran out (in which case it sets
// `*abort` itself); the caller then leaves its loop and falls through to the teardown.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();          // the SM cycle counter: reading %globaltimer costs far more
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort = 1;
        return false;
      }
    }
  }
}

// Warp-collective bounded wait: lane 0 polls; when it has seen the phase complete every lane
// performs one (immediately successful) try_wait of its own, which gives each lane the acquire
// it needs before touching the data, without 32 lanes hammering the barrier while it is pending.
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint64_t* bar, uint32_t parity, volatile int* abort) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_bounded(bar, parity, abort) ? 1 : 0;
  ok = __shfl_sync(0xFFFFFFFFu, ok, 0);
  if (ok) {
    while (!mbar_try_wait(bar, parity)) {
    }
  }
  return ok != 0;
}

// Tiled TMA loads for kernels that may run as a CTA pair.  CG = 2 uses the pair form of the
// instruction, whose completion bytes may be counted on an mbarrier of the other CTA of the
// pair: `bar_addr` is a shared::cluster address (clear bit 24 of a local address to name the
// even-ranked CTA's copy of the barrier).  Every CTA loads only its own tile.
template <int CG>
__device__ __forceinline__ void tma_load_2d_cg(uint32_t dst, const void* tmap, int32_t x, int32_t y, uint32_t bar_addr) {
  if constexpr (CG == 1)
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar_addr) : "memory");
  else
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar_addr) : "memory");
}
template <int CG>
__device__ __forceinline__ void tma_load_3d_cg(uint32_t dst, const void* tmap, int32_t x, int32_t y, int32_t z,
                                               uint32_t bar_addr) {
  if constexpr (CG == 1)
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
  else
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar_addr) : "memory");
}

__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// True in exactly one lane of a fully active warp.  Unlike `lane == 0`, the compiler knows the
// guarded code runs in a single lane, so the descriptor operands of TMA / tcgen05 instructions go
// to uniform registers directly instead of through a per-lane loop (measured: 3x cheaper issue).
__device__ __forceinline__ bool elect_one() {
  uint32_t p;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(p));
  return p != 0;
}
// warp index as a warp-uniform value
__device__ __forceinline__ int warp_index() { return __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0); }

// ---- cluster helpers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t nclusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
// arrive on an mbarrier given by a shared::cluster address (own or peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
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
// like mbar_wait_bounded, with cluster-scope acquire (the barrier is arrived on by the peer CTA)
__device__ __forceinline__ bool mbar_wait_bounded_cluster(uint64_t* bar, uint32_t parity, volatile int* abort) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();          // the SM cycle counter: reading %globaltimer costs far more
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((++spins & 63u) == 0) {
      if (*abort) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- tcgen05 ----------------------------------------------------------------------------
// CG = 1: one CTA per MMA; CG = 2: a CTA pair shares each MMA (cta_group::2).
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
                 "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
                 "r"(ncols) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CG == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on the mbarrier (shared::cluster address: own or peer CTA) when every tcgen05
// operation issued so far by this thread is done.
template <int CG>
__device__ __forceinline__ void tc_commit(uint32_t cluster_addr) {
  if constexpr (CG == 1)
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
  else
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
                 : "memory");
}
// The tcgen05 wrappers below take 64-bit shared-memory descriptors as two 32-bit words: only the low
// word (address field) changes between stages and K steps, so the issuing thread advances descriptors
// with 32-bit adds and the constant high word never moves.
#define PLQ_TC_MMA_ASM(CGSTR, KINDSTR)                                                                         \
  asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"                          \
               "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"                                          \
               "tcgen05.mma.cta_group::" CGSTR ".kind::" KINDSTR " [%0], da, db, %4, [%5], [%7], p;\n\t}" ::"r"( \
                   d_tmem),                                                                                    \
               "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(sfa_tmem), "r"(accumulate), "r"(sfb_tmem)   \
               : "memory")
template <int CG>
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  if constexpr (CG == 1) PLQ_TC_MMA_ASM("1", "mxf4nvf4.block_scale.block16");
  else PLQ_TC_MMA_ASM("2", "mxf4nvf4.block_scale.block16");
}
template <int CG>
__device__ __forceinline__ void tc_mma_mxf8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                            uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                            uint32_t accumulate) {
  if constexpr (CG == 1) PLQ_TC_MMA_ASM("1", "mxf8f6f4.block_scale");
  else PLQ_TC_MMA_ASM("2", "mxf8f6f4.block_scale");
}
#undef PLQ_TC_MMA_ASM
// Shared -> tensor memory copy of 32 rows x 128 bit, replicated to the four lane quadrants
// (for a CTA pair: in both CTAs, each from its own shared memory at the same offset).
template <int CG>
__device__ __forceinline__ void tc_cp_32x128b_warpx4(uint32_t taddr, uint32_t desc_lo, uint32_t desc_hi) {
  if constexpr (CG == 1)
    asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}" ::"r"(
                     taddr),
                 "r"(desc_lo), "r"(desc_hi)
                 : "memory");
  else
    asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\ttcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}" ::"r"(
                     taddr),
                 "r"(desc_lo), "r"(desc_hi)
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Programmatic dependent launch.  `pdl_launch_dependents`: the next kernel in the stream, if it was
// launched with programmatic stream serialisation, may start once every CTA of this grid has executed
// this (or exited).  `pdl_wait`: blocks until the preceding grid has completed and its writes are visible;
// everything a kernel does before it must not depend on, or disturb, earlier kernels.  Both are no-ops
// for ordinary launches.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// 32 lanes x 8 consecutive 32-bit columns
__device__ __forceinline__ void tc_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

#endif  // __CUDACC__
}  // namespace plq
