// Decode GEMV on the tensor cores, m <= 16:  Y[m, n] = deq(X)[m, :] . deq(W)[n, :]  (bf16 out)
//
// The weights are the M-side operand of the block-scaled MMA (128 weight rows per instruction)
// and the activations the N-side one (m rows, zero-filled to 16 by the TMA box), so the packed
// NVFP4 / MXFP8 weight bytes go HBM -> shared memory (TMA) -> tensor core and no thread ever
// touches, converts or scales them.  The kernel is bound by how fast the weight bytes stream in:
// a ring of four 22 KiB stages (16 KiB of weight codes, 2 KiB of weight scales, 2 + 2 KiB of
// activation codes and scales, which come from L2).  A CTA takes 104 KiB of shared memory so that two
// CTAs share an SM: ~176 KiB per SM in flight, and the CTAs of the next launch can set up and prefetch
// their weights while the previous launch's are still finishing.
//
// Work split.  A 128-row tile of W is the unit of output.  When there are fewer tiles than CTA slots,
// each tile is given to a thread-block cluster of S CTAs (S <= 4, all clusters resident
// at once), CTA r taking the r-th slice of the K stages; CTAs 1..S-1 push their float32 partial
// sums [8 or 16 activation rows, 128]
// into CTA 0's shared memory (distributed shared memory, one hop) and arrive on its barrier, and
// CTA 0 adds them in slice order (a fixed order: results do not depend on timing) and writes bf16.
// No scratch memory in HBM is needed.  Otherwise S = 1 and CTAs loop over whole tiles.
//
// Programmatic dependent launch: the kernel is launched so that it may start while the previous
// kernel in the stream drains.  Barrier set-up, tensor-memory allocation and descriptor prefetch
// happen before griddepcontrol.wait; every load and store after it - except
// that a caller who declares the weights static (flag PLQ_GEMV_STATIC_B) lets the first ring fill
// of weight bytes be requested before the wait.
//
//   warps 0, 2, 3  producers, stages round-robin (one thread each)
//   warp 1         MMA issuer: scale chunks shared -> tensor memory, four MMAs per stage
//   warps 4-7      epilogue: tensor memory -> registers -> output, or -> CTA 0 of the cluster
//
// Every wait is bounded; on expiry PLQ_DEV_TIMEOUT is stored to the caller's status word and
// all roles leave their loops (same protocol as the fused GEMM).
#include <cuda.h>
#include <cstring>

#include "plq_tc.cuh"

namespace plq {

constexpr int kGtN = 16;                                   // MMA N (activation rows, zero-filled)
constexpr int kGtXBytes = kGtN * kStageKBytes;             // 2 KiB
constexpr int kGtSfBytes = 4 * kSfChunk;                   // 2 KiB: four chunks of one 128-row group
constexpr int kGtStageBytes = kABytes + kGtXBytes + 2 * kGtSfBytes;
constexpr int kGtStagesAll = 4;                            // 4 x 22 KiB in flight per CTA; two CTAs share an SM
template <int MR> constexpr int kGtStagesFor = kGtStagesAll;
constexpr uint32_t kGtProducers = 3;                         // warps 0, 2, 3: one thread each, stages round-robin
constexpr int kGtAccStages = 2;
constexpr int kGtAccCols = 32;                             // spacing of the two accumulators (16 used)
constexpr int kGtSfCol0 = kGtAccStages * kGtAccCols;       // 64
constexpr int kGtSfSetCols = 32;                           // 4 MMAs x (4 weight + 4 activation columns)
constexpr int kGtTmemCols = 128;
constexpr int kGtThreads = 256;
constexpr int kGtEpiThreads = 128;
// K slices per tile = CTAs per cluster.  Bounded by the shared memory the partial-sum slots may take if two CTAs
// (of this launch, or the tail of one launch and the head of the next) are to fit one SM.
template <int MR> constexpr int kGtMaxSlicesFor = MR == 8 ? 4 : 3;
constexpr int kGtMaxSlices = 4;
template <int MR> constexpr int kGtSlotBytesFor = MR * 128 * 4;      // one partial: MR activation rows x 128 weight rows, float32
template <int MR>
constexpr size_t kGtSmemBytesFor = 1024 + static_cast<size_t>(kGtStagesFor<MR>) * kGtStageBytes + (kGtMaxSlicesFor<MR> - 1) * kGtSlotBytesFor<MR> + 512;
static_assert(kGtSfCol0 + 2 * kGtSfSetCols <= kGtTmemCols, "tensor memory budget");
static_assert(2 * (kGtSmemBytesFor<8> + 1024) <= 232448 && 2 * (kGtSmemBytesFor<16> + 1024) <= 232448,
              "two CTAs per SM (1 KiB per CTA is reserved by the system)");

struct GtMaps {
  CUtensorMap w_lo, x_lo, w_hi, x_hi, sfw_lo, sfx_lo, sfw_hi, sfx_hi;
};

#ifdef PLQ_GEMV_TRACE
// Debug builds only: every CTA stamps %globaltimer at its phase boundaries into trace[cta * 16 + phase].
#define PLQ_GT_STAMP(i) do { g.trace[static_cast<size_t>(blockIdx.x) * 16 + (i)] = globaltimer_ns(); } while (0)
#else
#define PLQ_GT_STAMP(i) do { } while (0)
#endif

struct GtArgs {
#ifdef PLQ_GEMV_TRACE
  unsigned long long* trace;
#endif
  __nv_bfloat16* y;
  int64_t ldy;
  int32_t* status;
  int m, n, k_lo, k_hi;
  int lo_stages, hi_stages, lo_chunks;
  int tiles;
  int static_b;                    // PLQ_GEMV_STATIC_B: weights may be loaded before the dependency wait
};

// and-reduction of a predicate over the 128 epilogue threads (named barrier 1)
__device__ __forceinline__ bool epi_all(bool ok) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 q, %1, 0;\n\tbar.red.and.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(ok))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

// MR = 8 or 16: how many activation rows (accumulator columns) the epilogue handles.
template <int MR>
__global__ void __launch_bounds__(kGtThreads, 2) gemv_tc_kernel(const __grid_constant__ GtMaps maps, const GtArgs g) {
  constexpr int kGtStages = kGtStagesFor<MR>;
  constexpr int kGtSlotBytes = kGtSlotBytesFor<MR>;
  constexpr int kGtSlotFloats = MR * 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* slots = reinterpret_cast<float*>(smem + static_cast<size_t>(kGtStages) * kGtStageBytes);   // CTA 0: partials of CTAs 1..S-1
  uint8_t* tail = reinterpret_cast<uint8_t*>(slots) + (kGtMaxSlicesFor<MR> - 1) * kGtSlotBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + kGtStages;
  uint64_t* acc_full = empty_bar + kGtStages;
  uint64_t* acc_empty = acc_full + kGtAccStages;
  uint64_t* red_bar = acc_empty + kGtAccStages;      // CTA 0: all partials of the tile have arrived
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(red_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = warp_index();
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) PLQ_GT_STAMP(0);                     // entry
  const int nslice = static_cast<int>(cluster_nctarank());   // S: CTAs sharing one tile along K
  const int slice = static_cast<int>(cluster_ctarank());

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGtStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kGtAccStages; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], kGtEpiThreads / 32);
    }
    mbar_init(red_bar, static_cast<uint32_t>(max(nslice - 1, 1)) * kGtEpiThreads);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && elect_one()) {
    if (g.k_lo) { prefetch_tmap(&maps.w_lo); prefetch_tmap(&maps.x_lo); prefetch_tmap(&maps.sfw_lo); prefetch_tmap(&maps.sfx_lo); }
    if (g.k_hi) { prefetch_tmap(&maps.w_hi); prefetch_tmap(&maps.x_hi); prefetch_tmap(&maps.sfw_hi); prefetch_tmap(&maps.sfx_hi); }
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_holder, kGtTmemCols);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  // CTA 0's barrier must be initialised before a peer arrives on it, which a peer does only at the very end of
  // its work: every CTA arrives on the cluster barrier here and waits on it just before its first remote access
  // (peers) or before it leaves (CTA 0), by which time the others have long arrived.
  if (nslice > 1) cluster_arrive_release();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  if (threadIdx.x == 0) PLQ_GT_STAMP(1);                     // barriers, tensor memory, cluster handshake done
  pdl_launch_dependents();          // the next kernel may be set up and prefetch its weights while this one runs

  // This CTA's work: K stages [ks_begin, ks_end) of tiles first_tile, first_tile + tile_step, ...
  // (a cluster of more than one CTA has exactly one tile: the host guarantees it).
  const int k_stages = g.lo_stages + g.hi_stages;
  const int ks_begin = (k_stages * slice) / nslice, ks_end = (k_stages * (slice + 1)) / nslice;
  const int first_tile = static_cast<int>(cluster_id_x()), tile_step = static_cast<int>(nclusters_x());
  const int my_tiles = first_tile < g.tiles ? (g.tiles - first_tile + tile_step - 1) / tile_step : 0;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0 || warp == 2 || warp == 3) {
    // ================================ producers ================================
    if (elect_one()) {
      const uint32_t pid = warp == 0 ? 0u : static_cast<uint32_t>(warp - 1);   // warps 0, 2, 3 -> 0, 1, 2
      auto issue = [&](uint32_t gs, int tile, int ks, bool w_part, bool x_part) {
        const uint32_t slot = gs % kGtStages;
        const bool lo = ks < g.lo_stages;
        const int kk = lo ? ks : ks - g.lo_stages;
        const int chunk0 = lo ? kk * 4 : kk;              // NVFP4: one chunk per MMA; MXFP8: one per stage
        const uint32_t st = smem_base + slot * kGtStageBytes;
        const uint32_t bar = smem_u32(&full_bar[slot]);
        if (w_part) {
          mbar_arrive_expect_tx(&full_bar[slot], kGtStageBytes);   // boxes always have their full size
          tma_load_2d_cg<1>(st, lo ? &maps.w_lo : &maps.w_hi, kk * kStageKBytes, tile * kBM, bar);
          tma_load_3d_cg<1>(st + kABytes + kGtXBytes, lo ? &maps.sfw_lo : &maps.sfw_hi, 0, chunk0, tile, bar);
        }
        if (x_part) {
          tma_load_2d_cg<1>(st + kABytes, lo ? &maps.x_lo : &maps.x_hi, kk * kStageKBytes, 0, bar);
          tma_load_3d_cg<1>(st + kABytes + kGtXBytes + kGtSfBytes, lo ? &maps.sfx_lo : &maps.sfx_hi, 0, chunk0, 0, bar);
        }
      };
      // By default both operands may have been written by the kernel just before this one (a weight packed right
      // before its first use included): nothing is loaded before the programmatic-dependency wait.  When the
      // caller declares the weights static (PLQ_GEMV_STATIC_B), the weight codes and scales of the first ring
      // fill are requested before the wait - they are in flight while the previous kernel drains - and the
      // activation parts of those stages after it.
      uint32_t n_init = 0;
      if (g.static_b) {
        n_init = min(static_cast<uint32_t>(my_tiles * (ks_end - ks_begin)), static_cast<uint32_t>(kGtStages));
        uint32_t gs0 = 0;
        for (int t = 0; t < my_tiles && gs0 < n_init; ++t)
          for (int ks = ks_begin; ks < ks_end && gs0 < n_init; ++ks, ++gs0)
            if (gs0 % kGtProducers == pid) issue(gs0, first_tile + t * tile_step, ks, true, false);
      }
      if (pid == 0) PLQ_GT_STAMP(2);                           // early weight loads issued
      pdl_wait();
      if (pid == 0) PLQ_GT_STAMP(3);                           // previous kernel complete
      if (g.static_b) {
        uint32_t gs0 = 0;
        for (int t = 0; t < my_tiles && gs0 < n_init; ++t)
          for (int ks = ks_begin; ks < ks_end && gs0 < n_init; ++ks, ++gs0)
            if (gs0 % kGtProducers == pid) issue(gs0, first_tile + t * tile_step, ks, false, true);
      }
      bool ok = true;
      uint32_t gs = 0;
      for (int t = 0; ok && t < my_tiles; ++t) {
        for (int ks = ks_begin; ks < ks_end; ++ks, ++gs) {
          if (gs % kGtProducers != pid || gs < n_init) continue;
          ok = mbar_wait_bounded(&empty_bar[gs % kGtStages], ((gs / kGtStages) & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          issue(gs, first_tile + t * tile_step, ks, true, true);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      // ================================ MMA issuer ================================
      constexpr uint32_t idesc_lo = make_idesc(1u /*E2M1*/, 128u, kGtN, 0u /*UE4M3*/);
      constexpr uint32_t idesc_hi = make_idesc(0u /*E4M3*/, 128u, kGtN, 1u /*UE8M0*/);
      const uint32_t a_lo0 = desc_lo_sw128(smem_base), b_lo0 = desc_lo_sw128(smem_base + kABytes);
      const uint32_t sf_lo0 = desc_lo_sf(smem_base + kABytes + kGtXBytes);
      constexpr uint32_t kStageStep = kGtStageBytes >> 4, kChunkStep = kSfChunk >> 4, kSfxOff = kGtSfBytes >> 4;
      int s = 0, as = 0;
      uint32_t phase = 0, aphase = 0, set = 0, soff = 0;
      bool ok = true;
      for (int t = 0; ok && t < my_tiles; ++t) {
        ok = mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * kGtAccCols;
        uint32_t accumulate = 0;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          ok = mbar_wait_bounded(&full_bar[s], phase, abort_flag);
          if (!ok) break;
          if (t == 0 && ks == ks_begin) PLQ_GT_STAMP(4);       // first stage landed
          tc_fence_after();
          const bool lo = ks < g.lo_stages;
          const int kk = lo ? ks : ks - g.lo_stages;
          const uint32_t sfw_t = tmem_base + kGtSfCol0 + set * kGtSfSetCols, sfx_t = sfw_t + 16;
          set ^= 1u;
          const uint32_t a_lo = a_lo0 + soff, b_lo = b_lo0 + soff, sf_lo = sf_lo0 + soff;
          const int nmma = lo ? min(4, g.lo_chunks - kk * 4) : min(4, (g.k_hi - kk * 128) / 32);
          if (lo && nmma == 4) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              tc_cp_32x128b_warpx4<1>(sfw_t + 4 * h, sf_lo + h * kChunkStep, kDescHiSf);
              tc_cp_32x128b_warpx4<1>(sfx_t + 4 * h, sf_lo + kSfxOff + h * kChunkStep, kDescHiSf);
            }
            tc_mma_nvf4<1>(d_tmem, a_lo, b_lo, kDescHiSw128, idesc_lo, sfw_t, sfx_t, accumulate);
#pragma unroll
            for (int h = 1; h < 4; ++h)
              tc_mma_nvf4<1>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc_lo, sfw_t + 4 * h, sfx_t + 4 * h, 1u);
          } else if (lo) {
            for (int h = 0; h < nmma; ++h) {
              tc_cp_32x128b_warpx4<1>(sfw_t + 4 * h, sf_lo + h * kChunkStep, kDescHiSf);
              tc_cp_32x128b_warpx4<1>(sfx_t + 4 * h, sf_lo + kSfxOff + h * kChunkStep, kDescHiSf);
            }
            for (int h = 0; h < nmma; ++h) {
              tc_mma_nvf4<1>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc_lo, sfw_t + 4 * h, sfx_t + 4 * h,
                             accumulate);
              accumulate = 1;
            }
          } else {
            // MXFP8: one chunk per stage, scale id h selects byte h of every scale column
            tc_cp_32x128b_warpx4<1>(sfw_t, sf_lo, kDescHiSf);
            tc_cp_32x128b_warpx4<1>(sfx_t, sf_lo + kSfxOff, kDescHiSf);
            for (int h = 0; h < nmma; ++h) {
              const uint32_t idesc = idesc_hi | (static_cast<uint32_t>(h) << 4) | (static_cast<uint32_t>(h) << 29);
              tc_mma_mxf8<1>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc,
                             sfw_t + (static_cast<uint32_t>(h) << 30), sfx_t + (static_cast<uint32_t>(h) << 30), accumulate);
              accumulate = 1;
            }
          }
          accumulate = 1;
          tc_commit<1>(smem_u32(&empty_bar[s]));       // stage reusable once these MMAs have read it
          soff += kStageStep;
          if (++s == kGtStages) { s = 0; soff = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit<1>(smem_u32(&acc_full[as]));
        if (t == my_tiles - 1) PLQ_GT_STAMP(5);                // last MMA issued
        if (++as == kGtAccStages) { as = 0; aphase ^= 1; }
      }
    }
  } else if (warp >= 4) {
    // ================================ epilogue ================================
    const int quad = warp & 3;                        // tensor-memory lane quadrant this warp may read
    const int trow = quad * 32 + lane;                // weight row inside the tile
    int as = 0;
    uint32_t aphase = 0;
    if (slice == 0) pdl_wait();                       // the output may still be in use by the previous kernel
    for (int t = 0; t < my_tiles; ++t) {
      bool ok = mbar_wait_bounded_warp(&acc_full[as], aphase, abort_flag);
      ok = epi_all(ok);                               // one decision for the four warps
      if (!ok) break;
      if (threadIdx.x == 128 && t == my_tiles - 1) PLQ_GT_STAMP(6);   // accumulator complete
      tc_fence_after();
      uint32_t r[MR];
      if constexpr (MR == 8) {
        tc_ld_32x32b_x8(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * kGtAccCols, r);
      } else {
        uint32_t h0[8], h1[8];
        tc_ld_32x32b_x8(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * kGtAccCols, h0);
        tc_ld_32x32b_x8(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * kGtAccCols + 8, h1);
#pragma unroll
        for (int j = 0; j < 8; ++j) { r[j] = h0[j]; r[8 + j] = h1[j]; }
      }
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
      if (++as == kGtAccStages) { as = 0; aphase ^= 1; }
      float acc[MR];
#pragma unroll
      for (int j = 0; j < MR; ++j) acc[j] = __uint_as_float(r[j]);
      if (slice > 0) {
        // push this slice's partial sums into CTA 0's slot (slice - 1), then arrive (release) on its barrier
        cluster_wait_acquire();                         // set-up of every CTA of the cluster is complete
        const uint32_t dst = map_to_cta(smem_u32(slots), 0u) + static_cast<uint32_t>((slice - 1) * kGtSlotBytes + trow * 4);
#pragma unroll
        for (int j = 0; j < MR; ++j) st_cluster_f32(dst + j * 512, acc[j]);
        mbar_arrive_cluster(map_to_cta(smem_u32(red_bar), 0u));
        if (threadIdx.x == 128) PLQ_GT_STAMP(7);            // partial pushed to CTA 0
        continue;
      }
      if (nslice > 1) {
        int got = 1;
        if (lane == 0) got = mbar_wait_bounded_cluster(red_bar, 0u, abort_flag) ? 1 : 0;
        got = __shfl_sync(0xFFFFFFFFu, got, 0);
        if (!epi_all(got != 0)) break;
        while (!mbar_try_wait_cluster(red_bar, 0u)) {   // completed: gives every thread the acquire
        }
        if (threadIdx.x == 128) PLQ_GT_STAMP(7);            // all partials have arrived
        for (int sl = 0; sl < nslice - 1; ++sl) {
#pragma unroll
          for (int j = 0; j < MR; ++j) acc[j] += slots[sl * kGtSlotFloats + j * 128 + trow];
        }
      }
      const int row = (first_tile + t * tile_step) * kBM + trow;
      if (row < g.n) {
#pragma unroll
        for (int j = 0; j < MR; ++j)
          if (j < g.m) g.y[static_cast<size_t>(j) * g.ldy + row] = __float2bfloat16_rn(acc[j]);
      }
      if (threadIdx.x == 128 && t == my_tiles - 1) PLQ_GT_STAMP(8);   // output stored
    }
  }

  // ================================ teardown ================================
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(g.status, PLQ_DEV_TIMEOUT);
    const long long t0 = clock64();                    // copies still in flight get time to land
    while (clock64() - t0 < 400000ll) __nanosleep(1000);
    __syncthreads();
  }
  // Only CTA 0's shared memory is written remotely, and CTA 0 has waited for every partial before it gets here:
  // nobody needs to wait for anybody to leave.  Threads that have not consumed the set-up phase of the cluster
  // barrier yet (everything but the epilogue warps of CTAs 1..) do it now; it completed long ago.
  if (nslice > 1 && !(slice > 0 && warp >= 4 && my_tiles > 0)) cluster_wait_acquire();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, kGtTmemCols);
  }
  if (threadIdx.x == 0) PLQ_GT_STAMP(9);                     // leaving
}

#ifdef PLQ_GEMV_TRACE
static unsigned long long* g_gt_trace = nullptr;   // set by plq_debug_set_gemv_trace; launch i writes at i * 148 * 16
static int g_gt_launch = 0;
#endif

// ---- host side --------------------------------------------------------------------------------
// How many clusters of each size the device can hold at once (one CTA per SM, clusters inside a GPC);
// looked up once per thread and device.
template <int MR>
static int gt_max_clusters(int slices) {
  static thread_local int cached_dev = -1;
  static thread_local int table[kGtMaxSlices + 1];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cached_dev != dev) {
    if (cudaFuncSetAttribute(gemv_tc_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kGtSmemBytesFor<MR>)) != cudaSuccess)
      return 0;
    for (int s = 1; s <= kGtMaxSlicesFor<MR>; ++s) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(s * 64), 1, 1);
      cfg.blockDim = dim3(kGtThreads, 1, 1);
      cfg.dynamicSmemBytes = kGtSmemBytesFor<MR>;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = static_cast<unsigned>(s);
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemv_tc_kernel<MR>, &cfg) != cudaSuccess) n = 0;
      table[s] = n;
    }
    (void)cudaGetLastError();
    cached_dev = dev;
  }
  return table[slices];
}

// K slices per tile (= cluster size) and grid: the largest slice count for which every tile's cluster is
// resident at once; one slice (CTAs looping over whole tiles) when there are more tiles than that.
template <int MR>
static void gt_plan(int64_t n, int64_t k_lo, int64_t k_hi, int sms, int* slices, int* grid) {
  const int tiles = static_cast<int>((n + kBM - 1) / kBM);
  const int k_stages = static_cast<int>((k_lo / 64 + 3) / 4 + (k_hi + 127) / 128);
  int s = (2 * sms) / tiles;                           // two CTAs fit an SM
  if (s > kGtMaxSlicesFor<MR>) s = kGtMaxSlicesFor<MR>;
  if (s > k_stages) s = k_stages;
  while (s > 1 && gt_max_clusters<MR>(s) < tiles) --s;
  if (s < 1) s = 1;
  *slices = s;
  *grid = s > 1 ? tiles * s : (tiles < 2 * sms ? tiles : 2 * sms);      // two CTAs fit an SM
}

template <int MR>
static int gt_launch(const GtMaps& tm, const GtArgs& g, int64_t n, int64_t k_lo, int64_t k_hi, cudaStream_t stream) {
  int slices = 1, grid = 1;
  if (gt_max_clusters<MR>(1) < 1) return PLQ_ERR_CUDA;     // also sets the kernel's shared-memory attribute
  gt_plan<MR>(n, k_lo, k_hi, sm_count(), &slices, &grid);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
  cfg.blockDim = dim3(kGtThreads, 1, 1);
  cfg.dynamicSmemBytes = kGtSmemBytesFor<MR>;
  cfg.stream = stream;
  // Programmatic dependent launch: this kernel may start while the previous one in the stream drains; it
  // touches nothing that depends on earlier work before its griddepcontrol.wait.
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = static_cast<unsigned>(slices);
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  PLQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_tc_kernel<MR>, tm, g));
  return PLQ_OK;
}

}  // namespace plq

extern "C" int plq_gemv_tc(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                           const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                           int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy,
                           int32_t* dev_status, int flags, void* stream) {
  using namespace plq;
  if (m < 1 || m > kGtN || n < 1 || k_lo < 0 || k_hi < 0 || k_lo + k_hi <= 0 || ldy < n) return PLQ_ERR_SHAPE;
  if (k_lo % 64 != 0 || k_hi % 32 != 0) return PLQ_ERR_SHAPE;
  if (n > (1 << 30) || k_lo > (1 << 24) || k_hi > (1 << 24)) return PLQ_ERR_LIMIT;
  if (!y_bf16 || !dev_status) return PLQ_ERR_NULL;
  if (k_lo && (!a_lo_codes || !a_lo_sf || !b_lo_codes || !b_lo_sf)) return PLQ_ERR_NULL;
  if (k_hi && (!a_hi_codes || !a_hi_sf || !b_hi_codes || !b_hi_sf)) return PLQ_ERR_NULL;
  if (!aligned16(a_lo_codes) || !aligned16(a_lo_sf) || !aligned16(a_hi_codes) || !aligned16(a_hi_sf) ||
      !aligned16(b_lo_codes) || !aligned16(b_lo_sf) || !aligned16(b_hi_codes) || !aligned16(b_hi_sf))
    return PLQ_ERR_ALIGN;
  int st = device_check();
  if (st != PLQ_OK) return st;

  GtArgs g;
  g.y = static_cast<__nv_bfloat16*>(y_bf16);
  g.ldy = ldy;
  g.status = dev_status;
  g.m = static_cast<int>(m); g.n = static_cast<int>(n);
  g.k_lo = static_cast<int>(k_lo); g.k_hi = static_cast<int>(k_hi);
  g.lo_chunks = static_cast<int>(k_lo / 64);
  g.lo_stages = (g.lo_chunks + 3) / 4;
  g.hi_stages = static_cast<int>((k_hi + 127) / 128);
  g.tiles = static_cast<int>((n + kBM - 1) / kBM);
  g.static_b = (flags & PLQ_GEMV_STATIC_B) ? 1 : 0;
#ifdef PLQ_GEMV_TRACE
  if (!g_gt_trace) return PLQ_ERR_NULL;
  g.trace = g_gt_trace + static_cast<size_t>(g_gt_launch++ % 64) * 256 * 16;
#endif

  GtMaps tm;
  memset(&tm, 0, sizeof(tm));
  const int64_t groups = (n + 127) / 128;
  if (k_lo) {
    if ((st = make_tmap(&tm.w_lo, b_lo_codes, n, k_lo / 2, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm.x_lo, a_lo_codes, m, k_lo / 2, kGtN)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfw_lo, b_lo_sf, g.lo_chunks, groups, 1)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfx_lo, a_lo_sf, g.lo_chunks, 1, 1)) != PLQ_OK) return st;
  }
  if (k_hi) {
    if ((st = make_tmap(&tm.w_hi, b_hi_codes, n, k_hi, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm.x_hi, a_hi_codes, m, k_hi, kGtN)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfw_hi, b_hi_sf, g.hi_stages, groups, 1)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfx_hi, a_hi_sf, g.hi_stages, 1, 1)) != PLQ_OK) return st;
  }
  return m <= 8 ? gt_launch<8>(tm, g, n, k_lo, k_hi, static_cast<cudaStream_t>(stream))
                : gt_launch<16>(tm, g, n, k_lo, k_hi, static_cast<cudaStream_t>(stream));
}

#ifdef PLQ_GEMV_TRACE
extern "C" __attribute__((visibility("default"))) void plq_debug_set_gemv_trace(void* buf) {
  plq::g_gt_trace = static_cast<unsigned long long*>(buf);
  plq::g_gt_launch = 0;
}
#endif
