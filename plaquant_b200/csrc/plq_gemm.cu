// Fused mixed NVFP4 / MXFP8 GEMM for sm_100a:  Y[m, n] = deq(A)[m, :] . deq(B)[n, :]  (bf16 out)
//
// One persistent, warp-specialised kernel.  Per output tile a single float32 accumulator lives
// in tensor memory; the NVFP4 K-range is issued as tcgen05.mma kind::mxf4nvf4 (K = 64 per
// instruction, four E4M3 scales per row) and the MXFP8 K-range as kind::mxf8f6f4 (K = 32 per
// instruction, one E8M0 scale per row) on top of the same columns.
//
// Two shapes of the same kernel (template parameter CG):
//   CG = 1  one CTA computes a 128 x BN tile.
//   CG = 2  a CTA pair (thread-block cluster of two, one TPC) computes a 256 x 256 tile with
//           tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and one half (128
//           rows) of B, so a CTA pulls 30 % fewer bytes from L2 per MMA.
//
//   warps 0, 2  producers, taking alternate K stages: TMA loads of the A/B code tiles (128-byte
//               swizzled rows, K-major) and bulk copies of the pre-tiled scale chunks into a ring of
//               shared-memory stages.  Two of them because one thread's issue rate (barrier wait,
//               expect-tx, five copy instructions: ~770 cycles measured) is longer than the 512
//               cycles the tensor pipe needs per stage.
//   warp 1      MMA issuer (leader CTA of a pair): copies the stage's scale chunks shared -> tensor
//               memory (tcgen05.cp), issues the MMAs, releases the stage and publishes finished
//               accumulators with tcgen05.commit.  In the second CTA of a pair this warp relays
//               "my stage has landed" to the leader.
//   warps 4+    epilogue: tcgen05.ld the accumulator to registers, release it, convert to bf16, store
//
// The single threads that issue TMA / tcgen05 instructions are chosen with elect.sync inside a
// warp-uniform branch: the compiler then keeps descriptors in uniform registers; with a plain
// `lane == 0` test the same instruction stream issued about three times slower (measured).
//
// A stage holds 128 bytes of K per row for both phases: 256 NVFP4 elements (four MMAs) or
// 128 MXFP8 elements (four MMAs).  Scale chunks are 512 bytes = 128 rows x 4 scales in the order
// tensor memory wants (row r -> lane r % 32, column r / 32, byte = scale index), so one
// tcgen05.cp.32x128b.warpx4 per chunk places them.
//
// Every mbarrier wait is bounded; on expiry the CTA records PLQ_DEV_TIMEOUT in the caller's
// status word, all roles leave their loops, outstanding copies get time to land, tensor memory
// is freed and the kernel returns.
#include <cuda.h>
#include <cstring>

#include "plq_tc.cuh"

namespace plq {

constexpr int kFirstEpiWarp = 4;
constexpr int kProducers = 2;

template <int BN, int CG>
struct GemmCfg {
  static_assert((BN == 128 && CG == 1) || BN == 256, "tile shapes: 128x128, 128x256, pair 256x256");
  static constexpr int kAccStages = BN == 128 ? 2 : 1;
  static constexpr int kEpiColSplit = BN == 128 ? 1 : 2;     // column groups handled by different warps
  static constexpr int kEpiWarps = 4 * kEpiColSplit;
  static constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
  static constexpr int kBRows = BN / CG;                     // B rows staged by one CTA
  static constexpr int kBBytes = kBRows * kStageKBytes;
  static constexpr int kSfGroups = BN / 128;                 // 128-row groups of B scales (all of them, in each CTA)
  static constexpr int kSfaBytes = 4 * kSfChunk;
  static constexpr int kSfbBytes = 4 * kSfChunk * kSfGroups;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = (BN == 128) ? 6 : (CG == 2 ? 5 : 4);
  static constexpr int kTmemCols = 512;
  static constexpr int kSfSetCols = 16 + 4 * (BN / 32);      // 4 MMAs x (4 A columns + BN/32 B columns)
  static constexpr int kSfSets = 2;                          // alternate per stage
  static constexpr int kSfCol0 = kAccStages * BN;
  static constexpr int kColsPerEpiWarp = BN / kEpiColSplit;  // 128
  static constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 512;
  static_assert(kSfCol0 + kSfSets * kSfSetCols <= kTmemCols, "tensor memory budget");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

struct GemmArgs {
  __nv_bfloat16* y;
  int64_t ldy;
  int32_t* status;
  int m, n, k_lo, k_hi;
  int tiles_m, tiles_n;            // tiles_m counts 128 * CG row tiles
  int lo_stages, hi_stages;        // K stages per tile in each phase
  int lo_chunks, hi_chunks;        // scale chunks per 128-row group
  int wide_store;                  // y and ldy allow 32-byte stores
  int band;                        // row tiles per band of the tile order
};

// Tile order: bands of `band` row tiles, inside a band M fastest, then N.  The CTAs that run at the same time
// then share `band` A tiles and (resident CTAs / band) B tiles instead of all A tiles and two or three B tiles.
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int band, int& tm, int& tn) {
  const int per_band = band * tiles_n;
  const int b = tile / per_band, r = tile - b * per_band;
  const int rows = min(band, tiles_m - b * band);          // the last band may be shorter
  tn = r / rows;
  tm = b * band + (r - tn * rows);
}

template <int BN, int CG>
__global__ void __launch_bounds__(GemmCfg<BN, CG>::kThreads, 1)
mixed_gemm_kernel(const __grid_constant__ GemmMaps maps, const GemmArgs g) {
  using C = GemmCfg<BN, CG>;
  const CUtensorMap& tm_a_lo = maps.a_lo;  const CUtensorMap& tm_b_lo = maps.b_lo;
  const CUtensorMap& tm_a_hi = maps.a_hi;  const CUtensorMap& tm_b_hi = maps.b_hi;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles (identical in both CTAs of a pair)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tail = smem + static_cast<size_t>(C::kStages) * C::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);      // stage landed (leader: in both CTAs) (1 + tx)
  uint64_t* empty_bar = full_bar + C::kStages;                // stage free                       (1 commit)
  uint64_t* acc_full = empty_bar + C::kStages;                 // accumulator complete             (1 commit)
  uint64_t* acc_empty = acc_full + C::kAccStages;              // leader: accumulator drained      (epi warps * CG)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + C::kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = warp_index();
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;      // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < C::kAccStages; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], C::kEpiWarps * CG);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && elect_one()) {
    if (g.k_lo) { prefetch_tmap(&tm_a_lo); prefetch_tmap(&tm_b_lo); prefetch_tmap(&maps.sfa_lo); prefetch_tmap(&maps.sfb_lo); }
    if (g.k_hi) { prefetch_tmap(&tm_a_hi); prefetch_tmap(&tm_b_hi); prefetch_tmap(&maps.sfa_hi); prefetch_tmap(&maps.sfb_hi); }
  }
  if (warp == 1) {
    tmem_alloc<CG>(tmem_holder, C::kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) {          // the peer's barriers must be initialised before anyone signals them
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_launch_dependents();          // the next kernel in the stream may be launched while this one runs

  const int num_tiles = g.tiles_m * g.tiles_n;
  const int k_stages = g.lo_stages + g.hi_stages;
  const int first_tile = CG == 2 ? static_cast<int>(cluster_id_x()) : static_cast<int>(blockIdx.x);
  const int tile_step = CG == 2 ? static_cast<int>(nclusters_x()) : static_cast<int>(gridDim.x);
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0 || warp == 2) {
    // ================================ producers ================================
    // Producer p takes the K stages whose running index (over all tiles of this CTA) is = p mod 2.
    if (elect_one()) {
      const int pid = warp == 0 ? 0 : 1;
      // One stage's loads.  In a pair every load of both CTAs is counted on the leader's barrier, which is the
      // one the MMA issuer waits on; boxes always have their full size (out-of-range parts are zero-filled).
      auto issue = [&](uint32_t gs, int tile, int ks) {
        int tm, tn;
        tile_coords(tile, g.tiles_m, g.tiles_n, g.band, tm, tn);
        const int mgrp = tm * CG + static_cast<int>(rank);        // this CTA's 128-row group of A
        const uint32_t slot = gs % C::kStages;
        const bool lo = ks < g.lo_stages;
        const int kk = lo ? ks : ks - g.lo_stages;
        const int chunk0 = lo ? kk * 4 : kk;              // NVFP4: one chunk per MMA; MXFP8: one per stage
        const uint32_t st = smem_base + slot * C::kStageBytes;
        const uint32_t bar = smem_u32(&full_bar[slot]) & (CG == 2 ? 0xFEFFFFFFu : 0xFFFFFFFFu);
        if (leader) mbar_arrive_expect_tx(&full_bar[slot], CG * C::kStageBytes);
        tma_load_2d_cg<CG>(st, lo ? &tm_a_lo : &tm_a_hi, kk * kStageKBytes, mgrp * kBM, bar);
        tma_load_2d_cg<CG>(st + kABytes, lo ? &tm_b_lo : &tm_b_hi, kk * kStageKBytes,
                           tn * BN + static_cast<int>(rank) * C::kBRows, bar);
        tma_load_3d_cg<CG>(st + kABytes + C::kBBytes, lo ? &maps.sfa_lo : &maps.sfa_hi, 0, chunk0, mgrp, bar);
        tma_load_3d_cg<CG>(st + kABytes + C::kBBytes + C::kSfaBytes, lo ? &maps.sfb_lo : &maps.sfb_hi, 0, chunk0,
                           tn * C::kSfGroups, bar);
      };
      // Stage gs (running over all tiles of this CTA) belongs to producer gs % 2.  Both operands may have been
      // written by the kernel just before this one (a weight packed right before its first use included), so
      // nothing is loaded before the programmatic-dependency wait; barrier set-up, tensor-memory allocation
      // and descriptor prefetch are what overlaps the previous kernel.
      pdl_wait();
      bool ok = true;
      uint32_t gs = pid;
      int tile = first_tile, ks = pid;
      while (ks >= k_stages && tile < num_tiles) { ks -= k_stages; tile += tile_step; }
      while (ok && tile < num_tiles) {
        for (; ks < k_stages; ks += kProducers, gs += kProducers) {
          ok = mbar_wait_bounded(&empty_bar[gs % C::kStages], ((gs / C::kStages) & 1u) ^ 1u, abort_flag);
          if (!ok) break;
          issue(gs, tile, ks);
        }
        ks -= k_stages;
        tile += tile_step;
        while (ks >= k_stages && tile < num_tiles) { ks -= k_stages; tile += tile_step; }
      }
    }
  } else if (warp == 1) {
    const bool elected = elect_one();
    if (elected && leader) {
      // ================================ MMA issuer ================================
      constexpr uint32_t idesc_lo = make_idesc(1u /*E2M1*/, 128u * CG, BN, 0u /*UE4M3*/);
      constexpr uint32_t idesc_hi = make_idesc(0u /*E4M3*/, 128u * CG, BN, 1u /*UE8M0*/);
      // barrier addresses to commit to: own CTA and, for a pair, the same barrier in the peer
      const uint32_t peer_off = CG == 2 ? map_to_cta(smem_u32(full_bar), 1u) - smem_u32(full_bar) : 0u;
      auto commit_all = [&](uint64_t* bar) {
        tc_commit<CG>(smem_u32(bar));
        if constexpr (CG == 2) tc_commit<CG>(smem_u32(bar) + peer_off);
      };
      // Descriptors as (low word, constant high word); the low word of stage s is base + s * stage bytes / 16.
      const uint32_t a_lo0 = desc_lo_sw128(smem_base), b_lo0 = desc_lo_sw128(smem_base + kABytes);
      const uint32_t sf_lo0 = desc_lo_sf(smem_base + kABytes + C::kBBytes);
      constexpr uint32_t kStageStep = C::kStageBytes >> 4, kChunkStep = kSfChunk >> 4, kSfbOff = C::kSfaBytes >> 4;
      int s = 0, as = 0;
      uint32_t phase = 0, aphase = 0, set = 0, soff = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        ok = CG == 2 ? mbar_wait_bounded_cluster(&acc_empty[as], aphase ^ 1, abort_flag)
                     : mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        uint32_t accumulate = 0;
        for (int ks = 0; ks < k_stages; ++ks) {
            ok = CG == 2 ? mbar_wait_bounded_cluster(&full_bar[s], phase, abort_flag)
                       : mbar_wait_bounded(&full_bar[s], phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const bool lo = ks < g.lo_stages;
          const int kk = lo ? ks : ks - g.lo_stages;
          const uint32_t sfa_t = tmem_base + C::kSfCol0 + set * C::kSfSetCols, sfb_t = sfa_t + 16;
          set ^= 1u;
          const uint32_t a_lo = a_lo0 + soff, b_lo = b_lo0 + soff, sf_lo = sf_lo0 + soff;
          const int nmma = lo ? min(4, g.lo_chunks - kk * 4) : min(4, (g.k_hi - kk * 128) / 32);
          // Scale chunks go shared -> tensor memory ahead of the MMAs that read them (the copies run
          // beside earlier MMAs in the tensor pipe).  The full stage is straight-line code with
          // immediate offsets: the issue rate of this one thread is what bounds the kernel otherwise.
          if (lo && nmma == 4) {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              tc_cp_32x128b_warpx4<CG>(sfa_t + 4 * h, sf_lo + h * kChunkStep, kDescHiSf);
#pragma unroll
              for (int q = 0; q < C::kSfGroups; ++q)
                tc_cp_32x128b_warpx4<CG>(sfb_t + (BN / 32) * h + 4 * q, sf_lo + kSfbOff + (q * 4 + h) * kChunkStep,
                                         kDescHiSf);
            }
            // advance 32 bytes (64 E2M1) inside the swizzle span: +2 in the address field
            tc_mma_nvf4<CG>(d_tmem, a_lo, b_lo, kDescHiSw128, idesc_lo, sfa_t, sfb_t, accumulate);
#pragma unroll
            for (int h = 1; h < 4; ++h)
              tc_mma_nvf4<CG>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc_lo, sfa_t + 4 * h,
                              sfb_t + (BN / 32) * h, 1u);
          } else if (lo) {
            for (int h = 0; h < nmma; ++h) {
              tc_cp_32x128b_warpx4<CG>(sfa_t + 4 * h, sf_lo + h * kChunkStep, kDescHiSf);
#pragma unroll
              for (int q = 0; q < C::kSfGroups; ++q)
                tc_cp_32x128b_warpx4<CG>(sfb_t + (BN / 32) * h + 4 * q, sf_lo + kSfbOff + (q * 4 + h) * kChunkStep,
                                         kDescHiSf);
            }
            for (int h = 0; h < nmma; ++h) {
              tc_mma_nvf4<CG>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc_lo, sfa_t + 4 * h,
                              sfb_t + (BN / 32) * h, accumulate);
              accumulate = 1;
            }
          } else {
            // MXFP8: one chunk per stage; scale id h selects byte h of every scale column (mirrored in
            // the top bits of the tensor-memory address)
            tc_cp_32x128b_warpx4<CG>(sfa_t, sf_lo, kDescHiSf);
#pragma unroll
            for (int q = 0; q < C::kSfGroups; ++q)
              tc_cp_32x128b_warpx4<CG>(sfb_t + 4 * q, sf_lo + kSfbOff + q * 4 * kChunkStep, kDescHiSf);
            for (int h = 0; h < nmma; ++h) {
              const uint32_t idesc = idesc_hi | (static_cast<uint32_t>(h) << 4) | (static_cast<uint32_t>(h) << 29);
              tc_mma_mxf8<CG>(d_tmem, a_lo + 2 * h, b_lo + 2 * h, kDescHiSw128, idesc,
                              sfa_t + (static_cast<uint32_t>(h) << 30), sfb_t + (static_cast<uint32_t>(h) << 30),
                              accumulate);
              accumulate = 1;
            }
          }
          accumulate = 1;
          commit_all(&empty_bar[s]);                 // stage reusable once these MMAs have read it
          soff += kStageStep;
          if (++s == C::kStages) { s = 0; soff = 0; phase ^= 1; }
        }
        if (!ok) break;
        commit_all(&acc_full[as]);                   // accumulator complete (in both CTAs of a pair)
        if (++as == C::kAccStages) { as = 0; aphase ^= 1; }
      }
    }
  } else if (warp >= kFirstEpiWarp) {
    // ================================ epilogue ================================
    const int e = warp - kFirstEpiWarp;
    const int quad = warp & 3;                      // tensor-memory lane quadrant this warp may read
    const int cgp = e >> 2;                         // column group
    const uint32_t empty_addr = CG == 2 ? map_to_cta(smem_u32(acc_empty), 0u) : smem_u32(acc_empty);
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    pdl_wait();                                       // the output may still be read by an earlier kernel
    for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
      int tm, tn;
      tile_coords(tile, g.tiles_m, g.tiles_n, g.band, tm, tn);
      const int row = (tm * CG + static_cast<int>(rank)) * kBM + quad * 32 + lane;
      const int col0 = tn * BN + cgp * C::kColsPerEpiWarp;
      ok = mbar_wait_bounded_warp(&acc_full[as], aphase, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * BN + cgp * C::kColsPerEpiWarp;
      // all loads first, one wait: the accumulator is handed back after a single tensor-memory round trip
      uint32_t r[C::kColsPerEpiWarp / 32][32];
#pragma unroll
      for (int c = 0; c < C::kColsPerEpiWarp / 32; ++c) tc_ld_32x32b_x32(taddr + c * 32, r[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty_addr + 8u * as);   // drained: the next tile may start
      if (++as == C::kAccStages) { as = 0; aphase ^= 1; }
      if (row < g.m) {
        // Streaming stores (the output is written once and not read by this kernel: keep L2 for the
        // operands), 32 bytes = one full sector per thread and instruction when the row allows it.
        __nv_bfloat16* yrow = g.y + static_cast<size_t>(row) * g.ldy;
        const bool wide = g.wide_store;
#pragma unroll
        for (int v = 0; v < C::kColsPerEpiWarp / 16; ++v) {
          const int col = col0 + v * 16;
          uint32_t d[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int cc = v * 16 + 2 * i;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;"
                : "=r"(d[i])
                : "f"(__uint_as_float(r[cc >> 5][(cc & 31) + 1])), "f"(__uint_as_float(r[cc >> 5][cc & 31])));
          }
          if (wide && col + 16 <= g.n) {
            asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(yrow + col), "r"(d[0]),
                         "r"(d[1]), "r"(d[2]), "r"(d[3]), "r"(d[4]), "r"(d[5]), "r"(d[6]), "r"(d[7])
                         : "memory");
          } else {
            if (col < g.n) __stcs(reinterpret_cast<uint4*>(yrow + col), make_uint4(d[0], d[1], d[2], d[3]));
            if (col + 8 < g.n) __stcs(reinterpret_cast<uint4*>(yrow + col + 8), make_uint4(d[4], d[5], d[6], d[7]));
          }
        }
      }
    }
  }

  // ================================ teardown ================================
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(g.status, PLQ_DEV_TIMEOUT);
    // give copies that are still in flight time to land before the shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);
    __syncthreads();
  }
  if constexpr (CG == 2) {          // the leader's MMAs read the peer's shared memory: leave together
    tc_fence_before();
    cluster_arrive_release();
    cluster_wait_acquire();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, C::kTmemCols);
  }
}

// ---- host side --------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// u8 matrix [rows, row_bytes], box = 128 bytes x box_rows, 128-byte swizzle, zero fill out of bounds.
int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return PLQ_ERR_TENSORMAP;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kStageKBytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? PLQ_OK : PLQ_ERR_TENSORMAP;
}

// Tiled scale buffer as int32 [128 words, chunks per group, groups]; box = 4 chunks of `box_groups` groups.
int make_sf_tmap(CUtensorMap* tm, const void* base, int64_t chunks, int64_t groups, int box_groups) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return PLQ_ERR_TENSORMAP;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(chunks), static_cast<cuuint64_t>(groups)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(kSfChunk), static_cast<cuuint64_t>(chunks) * kSfChunk};
  const cuuint32_t box[3] = {128, 4, static_cast<cuuint32_t>(box_groups)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? PLQ_OK : PLQ_ERR_TENSORMAP;
}

struct GemmPtrs {
  const void *a_lo, *a_lo_sf, *a_hi, *a_hi_sf, *b_lo, *b_lo_sf, *b_hi, *b_hi_sf;
};

template <int BN, int CG>
static int launch_gemm(const GemmPtrs& p, GemmArgs& g, cudaStream_t stream) {
  using C = GemmCfg<BN, CG>;
  GemmMaps tm;
  memset(&tm, 0, sizeof(tm));
  const int64_t mg = (g.m + 127) / 128, ng = (g.n + 127) / 128;
  int st;
  if (g.k_lo) {
    if ((st = make_tmap(&tm.a_lo, p.a_lo, g.m, g.k_lo / 2, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm.b_lo, p.b_lo, g.n, g.k_lo / 2, C::kBRows)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfa_lo, p.a_lo_sf, g.lo_chunks, mg, 1)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfb_lo, p.b_lo_sf, g.lo_chunks, ng, C::kSfGroups)) != PLQ_OK) return st;
  }
  if (g.k_hi) {
    if ((st = make_tmap(&tm.a_hi, p.a_hi, g.m, g.k_hi, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm.b_hi, p.b_hi, g.n, g.k_hi, C::kBRows)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfa_hi, p.a_hi_sf, g.hi_chunks, mg, 1)) != PLQ_OK) return st;
    if ((st = make_sf_tmap(&tm.sfb_hi, p.b_hi_sf, g.hi_chunks, ng, C::kSfGroups)) != PLQ_OK) return st;
  }
  g.tiles_m = (g.m + kBM * CG - 1) / (kBM * CG);
  g.tiles_n = (g.n + BN - 1) / BN;
  {
    // The operand that is walked in the inner direction is re-read once per step of the outer one and should
    // stay in L2.  M fastest (one band) re-reads A; when A is the larger operand and too big for that
    // (prefill down projection: 59 MB of A against 29 MB of B), narrow bands re-read B instead
    // (measured: 203 -> 187 us on that shape; 405 -> 446 us on gate_up, where B is the large one).
    const int64_t k_bytes = g.k_lo / 2 + g.k_hi;
    const int64_t a_bytes = static_cast<int64_t>(g.m) * k_bytes, b_bytes = static_cast<int64_t>(g.n) * k_bytes;
    g.band = (a_bytes > b_bytes && a_bytes > (32ll << 20)) ? 4 : g.tiles_m;
    if (g.band > g.tiles_m) g.band = g.tiles_m;
  }
  auto kernel = mixed_gemm_kernel<BN, CG>;
  static thread_local int attr_dev = -1;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    PLQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(C::kSmemBytes)));
    attr_dev = dev;
  }
  const int tiles = g.tiles_m * g.tiles_n;
  const int slots = sm_count() / CG;                 // CTAs (CG = 1) or CTA pairs (CG = 2) resident at once
  const int groups = tiles < slots ? tiles : slots;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(groups * CG), 1, 1);
  cfg.blockDim = dim3(C::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: set-up and the first weight loads may overlap the previous kernel's tail;
  // activations are read and the output written only after griddepcontrol.wait
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  PLQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tm, g));
  return PLQ_OK;
}

}  // namespace plq

extern "C" int plq_mixed_gemm_variant(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes,
                                   const void* a_hi_sf, const void* b_lo_codes, const void* b_lo_sf,
                                   const void* b_hi_codes, const void* b_hi_sf, int64_t m, int64_t n, int64_t k_lo,
                                   int64_t k_hi, void* y_bf16, int64_t ldy, int32_t* dev_status, void* stream,
                                   int variant) {
  using namespace plq;
  if (m < 1 || n < 1 || k_lo < 0 || k_hi < 0 || k_lo + k_hi <= 0) return PLQ_ERR_SHAPE;
  if (k_lo % 64 != 0 || k_hi % 32 != 0 || n % 8 != 0 || ldy % 8 != 0 || ldy < n) return PLQ_ERR_SHAPE;
  if (m > (1 << 30) || n > (1 << 30) || k_lo > (1 << 24) || k_hi > (1 << 24)) return PLQ_ERR_LIMIT;
  if (!y_bf16 || !dev_status) return PLQ_ERR_NULL;
  if (k_lo && (!a_lo_codes || !a_lo_sf || !b_lo_codes || !b_lo_sf)) return PLQ_ERR_NULL;
  if (k_hi && (!a_hi_codes || !a_hi_sf || !b_hi_codes || !b_hi_sf)) return PLQ_ERR_NULL;
  if (!aligned16(a_lo_codes) || !aligned16(a_lo_sf) || !aligned16(a_hi_codes) || !aligned16(a_hi_sf) ||
      !aligned16(b_lo_codes) || !aligned16(b_lo_sf) || !aligned16(b_hi_codes) || !aligned16(b_hi_sf) ||
      !aligned16(y_bf16))
    return PLQ_ERR_ALIGN;
  int st = device_check();
  if (st != PLQ_OK) return st;
  GemmArgs g;
  const GemmPtrs ptrs = {a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf};
  g.y = static_cast<__nv_bfloat16*>(y_bf16);
  g.ldy = ldy;
  g.status = dev_status;
  g.m = static_cast<int>(m); g.n = static_cast<int>(n);
  g.k_lo = static_cast<int>(k_lo); g.k_hi = static_cast<int>(k_hi);
  g.lo_chunks = static_cast<int>(k_lo / 64);
  g.hi_chunks = static_cast<int>((k_hi + 127) / 128);
  g.lo_stages = (g.lo_chunks + 3) / 4;
  g.hi_stages = g.hi_chunks;
  g.wide_store = (reinterpret_cast<uintptr_t>(y_bf16) % 32 == 0 && ldy % 16 == 0) ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (variant == PLQ_GEMM_AUTO) {
    // The kernel is bound by the bytes a CTA pulls from L2 per K stage (38 KB for a CTA of a pair, 54 KB
    // for a 128 x 256 tile, 36 KB for a 128 x 128 tile), so the cheapest shape is the one with the smallest
    // (waves over the SMs) x (bytes per stage); ties go to the larger tile.
    const int sms = sm_count();
    const int64_t mt = (m + 127) / 128;
    const int64_t pair_tiles = ((m + 255) / 256) * ((n + 255) / 256);
    const int64_t wide_tiles = mt * ((n + 255) / 256);
    const int64_t small_tiles = mt * ((n + 127) / 128);
    const int64_t pair_slots = sms / 2 > 0 ? sms / 2 : 1;
    const int64_t cost_pair = ((pair_tiles + pair_slots - 1) / pair_slots) * 38;
    const int64_t cost_wide = ((wide_tiles + sms - 1) / sms) * 54;
    const int64_t cost_small = ((small_tiles + sms - 1) / sms) * 36;
    variant = PLQ_GEMM_PAIR_256x256;
    int64_t best = cost_pair;
    if (cost_wide < best) { variant = PLQ_GEMM_128x256; best = cost_wide; }
    if (cost_small < best || n < 256) variant = PLQ_GEMM_128x128;
  }
  if (variant == PLQ_GEMM_128x128) return launch_gemm<128, 1>(ptrs, g, s);
  if (variant == PLQ_GEMM_128x256) return launch_gemm<256, 1>(ptrs, g, s);
  if (variant == PLQ_GEMM_PAIR_256x256) return launch_gemm<256, 2>(ptrs, g, s);
  return PLQ_ERR_SHAPE;
}

extern "C" int plq_mixed_gemm(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                              const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                              int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy,
                              int32_t* dev_status, void* stream) {
  return plq_mixed_gemm_variant(a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf,
                                m, n, k_lo, k_hi, y_bf16, ldy, dev_status, stream, PLQ_GEMM_AUTO);
}
