// Fused mixed NVFP4 / MXFP8 GEMM for sm_100a:  Y[m, n] = deq(A)[m, :] . deq(B)[n, :]  (bf16 out)
//
// One persistent, warp-specialised kernel.  Per 128 x BN output tile a single float32
// accumulator lives in tensor memory; the NVFP4 K-range is issued as tcgen05.mma
// kind::mxf4nvf4 (K = 64 per instruction, four E4M3 scales per row) and the MXFP8 K-range as
// kind::mxf8f6f4 (K = 32 per instruction, one E8M0 scale per row) on top of the same columns.
//
//   warp 0   producer: TMA loads of A/B code tiles (128-byte swizzled rows, K-major) and bulk
//            copies of the pre-tiled scale chunks into a ring of shared-memory stages
//   warp 1   MMA issuer: copies the scale chunks shared -> tensor memory (tcgen05.cp), issues
//            the MMAs, releases stages and publishes finished accumulators via tcgen05.commit
//   warps 4+ epilogue: tcgen05.ld the accumulator to registers, release it, convert to bf16, store
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

#include "plq_common.cuh"

namespace plq {

constexpr int kBM = 128;
constexpr int kStageKBytes = 128;                 // bytes of K per row per stage (one swizzle span)
constexpr int kABytes = kBM * kStageKBytes;       // 16 KiB
constexpr int kSfChunk = 512;
constexpr int kFirstEpiWarp = 4;

template <int BN>
struct GemmCfg {
  static_assert(BN == 128 || BN == 256, "tile N");
  static constexpr int kAccStages = BN == 128 ? 2 : 1;
  static constexpr int kEpiColSplit = BN == 128 ? 1 : 2;     // column groups handled by different warps
  static constexpr int kEpiWarps = 4 * kEpiColSplit;
  static constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
  static constexpr int kBBytes = BN * kStageKBytes;
  static constexpr int kSfaBytes = 4 * kSfChunk;             // four K chunks of 128 rows
  static constexpr int kSfbBytes = 4 * kSfChunk * (BN / 128);
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kStages = BN == 128 ? 6 : 4;
  static constexpr int kTmemCols = 512;
  static constexpr int kSfaCol = kAccStages * BN;            // 16 columns (4 MMAs x 4)
  static constexpr int kSfbCol = kSfaCol + 16;               // 4 MMAs x BN/32
  static constexpr int kColsPerEpiWarp = BN / kEpiColSplit;  // 128
  static constexpr size_t kSmemBytes = 1024 + static_cast<size_t>(kStages) * kStageBytes + 256;
  static_assert(kSfbCol + 4 * (BN / 32) <= kTmemCols, "tensor memory budget");
};

struct GemmArgs {
  const uint8_t* a_lo_sf;   // tiled
  const uint8_t* a_hi_sf;
  const uint8_t* b_lo_sf;
  const uint8_t* b_hi_sf;
  __nv_bfloat16* y;
  int64_t ldy;
  int32_t* status;
  int m, n, k_lo, k_hi;
  int tiles_m, tiles_n;
  int lo_stages, hi_stages;        // K stages per tile in each phase
  int lo_chunks, hi_chunks;        // scale chunks per 128-row group
  int n_sf_groups;                 // 128-row groups present in the B scale buffers
};

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 8-row
// groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_sw128_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);          // start address
  d |= static_cast<uint64_t>(1) << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                  // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                          // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                          // SWIZZLE_128B
  return d;
}
// Descriptor of one 512-byte scale chunk: 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// Instruction descriptor of a block-scaled MMA (M = 128, K-major operands).
//   [4,6) B scale id  [7,10) A format  [10,13) B format  [17,23) N/8  [23] scale format
//   [24,29) M/16  [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t n, uint32_t scale_is_e8m0) {
  return (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | (scale_is_e8m0 << 23) | ((128u >> 4) << 24);
}

template <int BN>
__global__ void __launch_bounds__(GemmCfg<BN>::kThreads, 1)
mixed_gemm_kernel(const __grid_constant__ CUtensorMap tm_a_lo, const __grid_constant__ CUtensorMap tm_b_lo,
                  const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_b_hi,
                  const GemmArgs g) {
  using C = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* tail = smem + static_cast<size_t>(C::kStages) * C::kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(tail);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full = empty_bar + C::kStages;
  uint64_t* acc_empty = acc_full + C::kAccStages;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + C::kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < C::kAccStages; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], C::kEpiWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0 && lane == 0) {
    if (g.k_lo) { prefetch_tmap(&tm_a_lo); prefetch_tmap(&tm_b_lo); }
    if (g.k_hi) { prefetch_tmap(&tm_a_hi); prefetch_tmap(&tm_b_hi); }
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int num_tiles = g.tiles_m * g.tiles_n;
  const int k_stages = g.lo_stages + g.hi_stages;

  auto stage_a = [&](int s) { return smem + static_cast<size_t>(s) * C::kStageBytes; };
  auto stage_b = [&](int s) { return stage_a(s) + kABytes; };
  auto stage_sfa = [&](int s) { return stage_b(s) + C::kBBytes; };
  auto stage_sfb = [&](int s) { return stage_sfa(s) + C::kSfaBytes; };

  if (warp == 0) {
    // ================================ producer ================================
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile % g.tiles_m, tn = tile / g.tiles_m;
        const int m0 = tm * kBM, n0 = tn * BN;
        for (int ks = 0; ks < k_stages; ++ks) {
          ok = mbar_wait_bounded(&empty_bar[s], phase ^ 1, abort_flag);
          if (!ok) break;
          const bool lo = ks < g.lo_stages;
          const int kk = lo ? ks : ks - g.lo_stages;
          // scale chunks of this stage: NVFP4 one per MMA (up to four), MXFP8 one per stage
          const int chunk0 = lo ? kk * 4 : kk;
          const int nchunk = lo ? min(4, g.lo_chunks - chunk0) : 1;
          const int chunks_k = lo ? g.lo_chunks : g.hi_chunks;
          const uint8_t* sfa = (lo ? g.a_lo_sf : g.a_hi_sf) + (static_cast<size_t>(tm) * chunks_k + chunk0) * kSfChunk;
          const uint8_t* sfb_base = lo ? g.b_lo_sf : g.b_hi_sf;
          int groups = 0;
          for (int h = 0; h < BN / 128; ++h) groups += (tn * (BN / 128) + h) < g.n_sf_groups;
          const uint32_t bytes = kABytes + C::kBBytes + static_cast<uint32_t>(nchunk) * kSfChunk * (1 + groups);
          mbar_arrive_expect_tx(&full_bar[s], bytes);
          tma_load_2d(stage_a(s), lo ? &tm_a_lo : &tm_a_hi, kk * kStageKBytes, m0, &full_bar[s]);
          tma_load_2d(stage_b(s), lo ? &tm_b_lo : &tm_b_hi, kk * kStageKBytes, n0, &full_bar[s]);
          bulk_g2s(stage_sfa(s), sfa, nchunk * kSfChunk, &full_bar[s]);
          for (int h = 0; h < BN / 128; ++h) {
            const int grp = tn * (BN / 128) + h;
            if (grp < g.n_sf_groups)
              bulk_g2s(stage_sfb(s) + h * 4 * kSfChunk,
                       sfb_base + (static_cast<size_t>(grp) * chunks_k + chunk0) * kSfChunk, nchunk * kSfChunk,
                       &full_bar[s]);
          }
          if (++s == C::kStages) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      constexpr uint32_t idesc_lo = make_idesc(1u /*E2M1*/, BN, 0u /*UE4M3*/);
      constexpr uint32_t idesc_hi = make_idesc(0u /*E4M3*/, BN, 1u /*UE8M0*/);
      const uint32_t sfa_t = tmem_base + C::kSfaCol;
      const uint32_t sfb_t = tmem_base + C::kSfbCol;
      int s = 0, as = 0;
      uint32_t phase = 0, aphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        ok = mbar_wait_bounded(&acc_empty[as], aphase ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + as * BN;
        uint32_t accumulate = 0;
        for (int ks = 0; ks < k_stages; ++ks) {
          ok = mbar_wait_bounded(&full_bar[s], phase, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const bool lo = ks < g.lo_stages;
          const int kk = lo ? ks : ks - g.lo_stages;
          const uint32_t a_addr = smem_u32(stage_a(s)), b_addr = smem_u32(stage_b(s));
          const uint32_t sfa_addr = smem_u32(stage_sfa(s)), sfb_addr = smem_u32(stage_sfb(s));
          const uint64_t adesc = make_sw128_desc(a_addr), bdesc = make_sw128_desc(b_addr);
          if (lo) {
            const int nmma = min(4, g.lo_chunks - kk * 4);
            for (int h = 0; h < nmma; ++h) {
              tc_cp_32x128b_warpx4(sfa_t + 4 * h, make_sf_desc(sfa_addr + h * kSfChunk));
#pragma unroll
              for (int q = 0; q < BN / 128; ++q)
                tc_cp_32x128b_warpx4(sfb_t + (BN / 32) * h + 4 * q, make_sf_desc(sfb_addr + (q * 4 + h) * kSfChunk));
            }
            for (int h = 0; h < nmma; ++h) {
              // advance 32 bytes (64 E2M1) inside the swizzle span: +2 in the address field
              tc_mma_nvf4(d_tmem, adesc + 2 * h, bdesc + 2 * h, idesc_lo, sfa_t + 4 * h, sfb_t + (BN / 32) * h,
                          accumulate);
              accumulate = 1;
            }
          } else {
            const int nmma = min(4, (g.k_hi - kk * 128) / 32);
            tc_cp_32x128b_warpx4(sfa_t, make_sf_desc(sfa_addr));
#pragma unroll
            for (int q = 0; q < BN / 128; ++q)
              tc_cp_32x128b_warpx4(sfb_t + 4 * q, make_sf_desc(sfb_addr + q * 4 * kSfChunk));
            for (int h = 0; h < nmma; ++h) {
              // scale id h selects byte h of every scale column; mirrored in the address' top bits
              const uint32_t idesc = idesc_hi | (static_cast<uint32_t>(h) << 4) | (static_cast<uint32_t>(h) << 29);
              tc_mma_mxf8(d_tmem, adesc + 2 * h, bdesc + 2 * h, idesc, sfa_t + (static_cast<uint32_t>(h) << 30),
                          sfb_t + (static_cast<uint32_t>(h) << 30), accumulate);
              accumulate = 1;
            }
          }
          tc_commit(&empty_bar[s]);                 // stage reusable once these MMAs have read it
          if (++s == C::kStages) { s = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&acc_full[as]);                   // accumulator complete
        if (++as == C::kAccStages) { as = 0; aphase ^= 1; }
      }
    }
  } else if (warp >= kFirstEpiWarp) {
    // ================================ epilogue ================================
    const int e = warp - kFirstEpiWarp;
    const int quad = warp & 3;                      // tensor-memory lane quadrant this warp may read
    const int cgp = e >> 2;                         // column group
    int as = 0;
    uint32_t aphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm = tile % g.tiles_m, tn = tile / g.tiles_m;
      const int row = tm * kBM + quad * 32 + lane;
      const int col0 = tn * BN + cgp * C::kColsPerEpiWarp;
      ok = mbar_wait_bounded(&acc_full[as], aphase, abort_flag);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + as * BN + cgp * C::kColsPerEpiWarp;
      uint32_t packed[C::kColsPerEpiWarp / 2];
#pragma unroll
      for (int c = 0; c < C::kColsPerEpiWarp / 32; ++c) {
        uint32_t r[32];
        tc_ld_32x32b_x32(taddr + c * 32, r);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          uint32_t d;
          asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(__uint_as_float(r[2 * i + 1])), "f"(__uint_as_float(r[2 * i])));
          packed[c * 16 + i] = d;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);   // accumulator drained: the next tile may start
      if (++as == C::kAccStages) { as = 0; aphase ^= 1; }
      if (row < g.m) {
        __nv_bfloat16* yrow = g.y + static_cast<size_t>(row) * g.ldy;
#pragma unroll
        for (int v = 0; v < C::kColsPerEpiWarp / 8; ++v) {
          const int col = col0 + v * 8;
          if (col < g.n)
            *reinterpret_cast<uint4*>(yrow + col) =
                make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
        }
      }
    }
  }

  // ================================ teardown ================================
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) atomicExch(g.status, PLQ_DEV_TIMEOUT);
    // give copies that are still in flight time to land before the shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
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
static int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
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

template <int BN>
static int launch_gemm(const void* a_lo, const void* a_hi, const void* b_lo, const void* b_hi, GemmArgs& g,
                       cudaStream_t stream) {
  using C = GemmCfg<BN>;
  CUtensorMap tm_a_lo, tm_b_lo, tm_a_hi, tm_b_hi;
  memset(&tm_a_lo, 0, sizeof(CUtensorMap)); memset(&tm_b_lo, 0, sizeof(CUtensorMap));
  memset(&tm_a_hi, 0, sizeof(CUtensorMap)); memset(&tm_b_hi, 0, sizeof(CUtensorMap));
  int st;
  if (g.k_lo) {
    if ((st = make_tmap(&tm_a_lo, a_lo, g.m, g.k_lo / 2, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm_b_lo, b_lo, g.n, g.k_lo / 2, BN)) != PLQ_OK) return st;
  }
  if (g.k_hi) {
    if ((st = make_tmap(&tm_a_hi, a_hi, g.m, g.k_hi, kBM)) != PLQ_OK) return st;
    if ((st = make_tmap(&tm_b_hi, b_hi, g.n, g.k_hi, BN)) != PLQ_OK) return st;
  }
  g.tiles_m = (g.m + kBM - 1) / kBM;
  g.tiles_n = (g.n + BN - 1) / BN;
  static thread_local int attr_dev = -1;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    PLQ_CUDA_TRY(cudaFuncSetAttribute(mixed_gemm_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(C::kSmemBytes)));
    attr_dev = dev;
  }
  const int tiles = g.tiles_m * g.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  mixed_gemm_kernel<BN><<<grid, C::kThreads, C::kSmemBytes, stream>>>(tm_a_lo, tm_b_lo, tm_a_hi, tm_b_hi, g);
  PLQ_CUDA_TRY(cudaGetLastError());
  return PLQ_OK;
}

}  // namespace plq

extern "C" int plq_mixed_gemm_tile(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes,
                                   const void* a_hi_sf, const void* b_lo_codes, const void* b_lo_sf,
                                   const void* b_hi_codes, const void* b_hi_sf, int64_t m, int64_t n, int64_t k_lo,
                                   int64_t k_hi, void* y_bf16, int64_t ldy, int32_t* dev_status, void* stream,
                                   int tile_n) {
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
  g.a_lo_sf = static_cast<const uint8_t*>(a_lo_sf); g.a_hi_sf = static_cast<const uint8_t*>(a_hi_sf);
  g.b_lo_sf = static_cast<const uint8_t*>(b_lo_sf); g.b_hi_sf = static_cast<const uint8_t*>(b_hi_sf);
  g.y = static_cast<__nv_bfloat16*>(y_bf16);
  g.ldy = ldy;
  g.status = dev_status;
  g.m = static_cast<int>(m); g.n = static_cast<int>(n);
  g.k_lo = static_cast<int>(k_lo); g.k_hi = static_cast<int>(k_hi);
  g.lo_chunks = static_cast<int>(k_lo / 64);
  g.hi_chunks = static_cast<int>((k_hi + 127) / 128);
  g.lo_stages = (g.lo_chunks + 3) / 4;
  g.hi_stages = g.hi_chunks;
  g.n_sf_groups = static_cast<int>((n + 127) / 128);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tile_n == 128) return launch_gemm<128>(a_lo_codes, a_hi_codes, b_lo_codes, b_hi_codes, g, s);
  if (tile_n == 256) return launch_gemm<256>(a_lo_codes, a_hi_codes, b_lo_codes, b_hi_codes, g, s);
  return PLQ_ERR_SHAPE;
}

extern "C" int plq_mixed_gemm(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                              const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                              int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy,
                              int32_t* dev_status, void* stream) {
  // Wide tiles halve the shared-memory traffic per MMA; narrow ones give small problems more CTAs.
  const int64_t tiles256 = ((m + 127) / 128) * ((n + 255) / 256);
  const int tile_n = (tiles256 >= plq::sm_count() || n % 256 == 0) && n >= 256 ? 256 : 128;
  return plq_mixed_gemm_tile(a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf, m,
                             n, k_lo, k_hi, y_bf16, ldy, dev_status, stream, tile_n);
}
