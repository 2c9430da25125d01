// Decode GEMV for m <= 8 tokens: y[m, n] = deq(A)[m, :] . deq(B)[n, :], HBM-bound on B.
//
// The weights are streamed exactly once; each warp owns 16 weight rows at a time and uses the
// warp-level m16n8k16 f16 MMA as its dot-product engine (A fragment = 16 weight rows, B fragment
// = the <= 8 activation rows), because eight tokens times ~7 CUDA-core operations per weight
// element would not keep up with HBM.  Products are exact in f16 (E2M1 x E4M3 and E4M3 values are
// f16-representable), accumulation is float32.
//
//   * Persistent grid, one CTA per SM.  Work unit = (16-row tile, K slice); K is cut into
//     `k_slices` slices so that every SM gets ~8-16 units, one per warp, whatever N is.  CTA b owns
//     slice b % k_slices and dequantises only that slice of the activations into shared memory,
//     once, already arranged in B-fragment order.
//   * Each lane streams its own bytes through a private cp.async ring (depth D chunks of 128
//     elements): lane (g = lane / 4, t = lane % 4) fetches the 16 bytes holding elements
//     32t .. 32t+31 of rows g and g+8, and reads back only what it wrote, so the ring needs no
//     block-level synchronisation and keeps D x 1 KiB per warp in flight while earlier chunks are
//     being multiplied.
//   * The MMA sums over K, so which K elements sit in which fragment slot is free as long as both
//     operands agree: MMA number j of a chunk consumes elements 32t + 4j .. 32t + 4j + 3 of every
//     lane.  No cross-lane shuffle of weight data.
//   * NVFP4 scales are folded into the f16 operands (exact); MXFP8 scales are powers of two applied
//     in float32 after the two MMAs of a 32-element block.
//   * With more than one K slice, partial sums go to a float32 scratch buffer; the warp that
//     delivers the last slice of a tile (an atomic ticket per tile) adds them in slice order, so
//     the result does not depend on timing, writes y and resets the ticket.
#include <atomic>
#include "plq_quant.cuh"

namespace plq {

struct GemvArgs {
  const uint8_t *a_lo, *a_lo_sf, *a_hi, *a_hi_sf;   // activations, m rows, row-major scales
  const uint8_t *b_lo, *b_lo_sf, *b_hi, *b_hi_sf;   // weights, n rows, row-major scales
  int m, n, k_lo, k_hi;
  __nv_bfloat16* y;
  int64_t ldy;
  int k_slices, cps, hps;   // lo chunks (128 elements) and hi blocks (32 elements) per slice
  int tiles;                // 16-row tiles
  float* partial;           // [k_slices][tiles * 16][8] float32 (k_slices > 1)
  unsigned int* tickets;    // [tiles], zero between calls
};

constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kGemvParts = 1;                     // warps sharing one 16-row tile (halves of the K slice)
constexpr int kGemvRedBytes = 2 * kGemvWarps * 128 * 4;   // double-buffered partial accumulators
constexpr int kRingStageBytes = 1024 + 128;       // 2 rows x 32 lanes x 16 B of codes + 16 rows x 8 B of scales

// Eight E2M1 codes (one 32-bit word, element 0 in bits [0,4)) -> four f16x2 registers:
// d0 = elements (0,1), d1 = (2,3), d2 = (4,5), d3 = (6,7).
__device__ __forceinline__ void cvt_e2m1x8_to_f16x2(uint32_t w, uint32_t& d0, uint32_t& d1, uint32_t& d2,
                                                    uint32_t& d3) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
      : "r"(w));
}
__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint32_t half16) {
  uint32_t d;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(d) : "h"(static_cast<uint16_t>(half16)));
  return d;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int D>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* xs_lo = reinterpret_cast<uint4*>(smem);                          // [cps][4][32] x 8 f16
  uint4* xs_hi = xs_lo + a.cps * 128;                                      // [hps][32] x 8 f16
  float* sxh = reinterpret_cast<float*>(xs_hi + a.hps * 32);               // [hps][8]
  uint8_t* rings = reinterpret_cast<uint8_t*>(sxh + a.hps * 8);            // [warps][D] ring stages

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.x % a.k_slices;
  const int cta_in_slice = blockIdx.x / a.k_slices;
  const int ctas_in_slice = (gridDim.x - slice + a.k_slices - 1) / a.k_slices;

  const int total_chunks = (a.k_lo + 127) >> 7;
  const int c_begin = min(slice * a.cps, total_chunks);
  const int c_end = min(c_begin + a.cps, total_chunks);
  const int nchunks_slice = c_end - c_begin;
  // kGemvParts warps may share a tile, each streaming a contiguous part of the slice's chunks and adding
  // their parts through shared memory (measured slower than one warp per tile on B200, so it is 1).
  const int part = warp & (kGemvParts - 1), slot = warp / kGemvParts;
  const int cpp = (nchunks_slice + kGemvParts - 1) / kGemvParts;
  const int p_begin = min(part * cpp, nchunks_slice);           // first chunk of this warp, relative to c_begin
  const int nchunks = min(cpp, nchunks_slice - p_begin);
  const int total_hb = a.k_hi >> 5;
  const int h_begin = min(slice * a.hps, total_hb);
  const int h_end = min(h_begin + a.hps, total_hb);

  // ---- this warp's ring: per stage [2 rows][32 lanes] x 16 B of codes, then [16 rows] x 8 B of scales ----
  uint8_t* ring = rings + static_cast<size_t>(warp) * D * kRingStageBytes;
  const uint32_t ring_u32 = smem_u32(ring);
  const bool lane_ok_base = true;
  (void)lane_ok_base;

  // per-tile state, set by `open_tile`
  int tile = 0, row_a = 0, row_b = 0, ra = 0, rb = 0;
  const uint8_t *wa = nullptr, *wb = nullptr, *sa = nullptr, *sb = nullptr;
  auto open_tile = [&](int q) -> bool {
    tile = cta_in_slice + ctas_in_slice * q;
    if (tile >= a.tiles) return false;
    row_a = tile * 16 + g; row_b = row_a + 8;
    ra = min(row_a, a.n - 1); rb = min(row_b, a.n - 1);
    wa = a.b_lo + static_cast<size_t>(ra) * (a.k_lo >> 1) + t * 16;
    wb = a.b_lo + static_cast<size_t>(rb) * (a.k_lo >> 1) + t * 16;
    sa = a.b_lo_sf + static_cast<size_t>(ra) * (a.k_lo >> 4) + t * 2;   // t even: 4 bytes from here
    sb = a.b_lo_sf + static_cast<size_t>(rb) * (a.k_lo >> 4) + t * 2;
    return true;
  };
  auto issue = [&](int i) {             // chunk i of the slice -> ring stage i % D
    const int c = c_begin + p_begin + i;
    if (c * 128 + t * 32 < a.k_lo) {
      const uint32_t st = ring_u32 + (i % D) * kRingStageBytes;
      cp_async_16(st + lane * 16, wa + c * 64);
      cp_async_16(st + 512 + lane * 16, wb + c * 64);
      if ((t & 1) == 0) {
        cp_async_4(st + 1024 + g * 8 + t * 2, sa + c * 8);
        cp_async_4(st + 1024 + (g + 8) * 8 + t * 2, sb + c * 8);
      }
    }
  };
  auto prime = [&]() {                  // first D-1 chunks of the current tile in flight
#pragma unroll
    for (int i = 0; i < D - 1; ++i) {
      if (i < nchunks) issue(i);
      cp_async_commit();
    }
  };
  // The first tile's weights start streaming before the activations are staged: they do not depend on them.
  bool have_tile = open_tile(slot);
  if (have_tile) prime();

  // ---- stage this CTA's K slice of the activations, dequantised, in fragment order ------------
  {
    const int units = nchunks_slice * 16;                // 8-element units per row in this slice
#pragma unroll 4
    for (int it = tid; it < units * 8; it += kGemvThreads) {
      const int row = it / units, u = it - row * units;
      const int c = u >> 4, tt = (u >> 2) & 3, jj = u & 3;
      const int k = (c_begin + c) * 128 + tt * 32 + jj * 8;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (row < a.m && k < a.k_lo) {
        const uint32_t codes = *reinterpret_cast<const uint32_t*>(a.a_lo + (static_cast<size_t>(row) * a.k_lo + k) / 2);
        const uint32_t sc = a.a_lo_sf[static_cast<size_t>(row) * (a.k_lo >> 4) + (k >> 4)];
        const uint32_t s2 = cvt_e4m3x2_to_f16x2(sc | (sc << 8));
        cvt_e2m1x8_to_f16x2(codes, o.x, o.y, o.z, o.w);
        o.x = hmul2_u32(o.x, s2); o.y = hmul2_u32(o.y, s2);
        o.z = hmul2_u32(o.z, s2); o.w = hmul2_u32(o.w, s2);
      }
      xs_lo[(c * 4 + jj) * 32 + row * 4 + tt] = o;
    }
    const int hunits = (h_end - h_begin) * 4;
    for (int it = tid; it < hunits * 8; it += kGemvThreads) {
      const int row = it / hunits, u = it - row * hunits;
      const int hb = u >> 2, tt = u & 3;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (row < a.m) {
        const uint2 codes = *reinterpret_cast<const uint2*>(a.a_hi + static_cast<size_t>(row) * a.k_hi +
                                                            (h_begin + hb) * 32 + tt * 8);
        o.x = cvt_e4m3x2_to_f16x2(codes.x & 0xFFFF); o.y = cvt_e4m3x2_to_f16x2(codes.x >> 16);
        o.z = cvt_e4m3x2_to_f16x2(codes.y & 0xFFFF); o.w = cvt_e4m3x2_to_f16x2(codes.y >> 16);
      }
      xs_hi[hb * 32 + row * 4 + tt] = o;
    }
    for (int it = tid; it < (h_end - h_begin) * 8; it += kGemvThreads) {
      const int hb = it >> 3, row = it & 7;
      sxh[it] = row < a.m ? e8m0_to_f32(a.a_hi_sf[static_cast<size_t>(row) * (a.k_hi >> 5) + h_begin + hb]) : 0.0f;
    }
  }
  __syncthreads();

  float* red = reinterpret_cast<float*>(rings + static_cast<size_t>(kGemvWarps) * D * kRingStageBytes);   // [2][slots][parts][32][4]
  int round = 0;
  for (int q = slot; have_tile; ) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float acc2[4] = {0.0f, 0.0f, 0.0f, 0.0f};          // second chain: consecutive MMAs do not depend on each other
    for (int i = 0; i < nchunks; ++i) {
      if (i + D - 1 < nchunks) issue(i + D - 1);
      cp_async_commit();
      cp_async_wait<D - 1>();
      __syncwarp();
      const int c = c_begin + p_begin + i;
      const uint8_t* st = ring + (i % D) * kRingStageBytes;
      uint4 va = make_uint4(0, 0, 0, 0), vb = va;
      uint32_t fa = 0, fb = 0;
      if (c * 128 + t * 32 < a.k_lo) {
        va = *reinterpret_cast<const uint4*>(st + lane * 16);
        vb = *reinterpret_cast<const uint4*>(st + 512 + lane * 16);
        fa = *reinterpret_cast<const uint16_t*>(st + 1024 + g * 8 + t * 2);
        fb = *reinterpret_cast<const uint16_t*>(st + 1024 + (g + 8) * 8 + t * 2);
      }
      const uint32_t sfa = cvt_e4m3x2_to_f16x2(fa), sfb = cvt_e4m3x2_to_f16x2(fb);
      const uint32_t sa0 = __byte_perm(sfa, sfa, 0x1010), sa1 = __byte_perm(sfa, sfa, 0x3232);
      const uint32_t sb0 = __byte_perm(sfb, sfb, 0x1010), sb1 = __byte_perm(sfb, sfb, 0x3232);
      const uint32_t wva[4] = {va.x, va.y, va.z, va.w};
      const uint32_t wvb[4] = {vb.x, vb.y, vb.z, vb.w};
      const uint4* xrow = xs_lo + (p_begin + i) * 128 + lane;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint4 xb = xrow[jj * 32];
        const uint32_t scale_a = jj < 2 ? sa0 : sa1, scale_b = jj < 2 ? sb0 : sb1;
        uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
        cvt_e2m1x8_to_f16x2(wva[jj], a0, a2, e0, e2);
        cvt_e2m1x8_to_f16x2(wvb[jj], a1, a3, e1, e3);
        mma_16816(acc, hmul2_u32(a0, scale_a), hmul2_u32(a1, scale_b), hmul2_u32(a2, scale_a),
                  hmul2_u32(a3, scale_b), xb.x, xb.y);
        mma_16816(acc2, hmul2_u32(e0, scale_a), hmul2_u32(e1, scale_b), hmul2_u32(e2, scale_a),
                  hmul2_u32(e3, scale_b), xb.z, xb.w);
      }
      __syncwarp();                      // all lanes done with this stage before it is refilled
    }
    cp_async_wait<0>();

    // ---- MXFP8 outlier columns of this slice ----
    for (int hb = h_begin + part; hb < h_end; hb += kGemvParts) {
      const uint2 ca = __ldcs(reinterpret_cast<const uint2*>(a.b_hi + static_cast<size_t>(ra) * a.k_hi + hb * 32 + t * 8));
      const uint2 cb = __ldcs(reinterpret_cast<const uint2*>(a.b_hi + static_cast<size_t>(rb) * a.k_hi + hb * 32 + t * 8));
      const float swa = e8m0_to_f32(a.b_hi_sf[static_cast<size_t>(ra) * (a.k_hi >> 5) + hb]);
      const float swb = e8m0_to_f32(a.b_hi_sf[static_cast<size_t>(rb) * (a.k_hi >> 5) + hb]);
      const uint4 xb = xs_hi[(hb - h_begin) * 32 + lane];
      float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      mma_16816(tmp, cvt_e4m3x2_to_f16x2(ca.x & 0xFFFF), cvt_e4m3x2_to_f16x2(cb.x & 0xFFFF),
                cvt_e4m3x2_to_f16x2(ca.x >> 16), cvt_e4m3x2_to_f16x2(cb.x >> 16), xb.x, xb.y);
      mma_16816(tmp, cvt_e4m3x2_to_f16x2(ca.y & 0xFFFF), cvt_e4m3x2_to_f16x2(cb.y & 0xFFFF),
                cvt_e4m3x2_to_f16x2(ca.y >> 16), cvt_e4m3x2_to_f16x2(cb.y >> 16), xb.z, xb.w);
      const float sx0 = sxh[(hb - h_begin) * 8 + 2 * t], sx1 = sxh[(hb - h_begin) * 8 + 2 * t + 1];
      acc[0] = fmaf(tmp[0], swa * sx0, acc[0]);
      acc[1] = fmaf(tmp[1], swa * sx1, acc[1]);
      acc[2] = fmaf(tmp[2], swb * sx0, acc[2]);
      acc[3] = fmaf(tmp[3], swb * sx1, acc[3]);
    }

    // ---- add the two halves of the tile (fixed order), in the warp with part 0 ----
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
    if constexpr (kGemvParts > 1) {
      float* r = red + ((static_cast<size_t>(round & 1) * (kGemvWarps / kGemvParts) + slot) * kGemvParts) * 128;
      if (part != 0) *reinterpret_cast<float4*>(r + part * 128 + lane * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      asm volatile("bar.sync %0, %1;" ::"r"(slot + 1), "r"(kGemvParts * 32) : "memory");
      if (part == 0) {
#pragma unroll
        for (int pp = 1; pp < kGemvParts; ++pp) {
          const float4 o = *reinterpret_cast<const float4*>(r + pp * 128 + lane * 4);
          acc[0] += o.x; acc[1] += o.y; acc[2] += o.z; acc[3] += o.w;
        }
      }
    }
    ++round;
    // ---- combine the K slices and store: lane holds (row g | g+8, tokens 2t | 2t+1) ----
    const int col = 2 * t;
    bool write_out = part == 0;
    if (a.k_slices > 1 && part == 0) {
      float* mine = a.partial + (static_cast<size_t>(slice) * a.tiles + tile) * 128;
      *reinterpret_cast<float2*>(mine + g * 8 + col) = make_float2(acc[0], acc[1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * 8 + col) = make_float2(acc[2], acc[3]);
      __threadfence();
      __syncwarp();
      unsigned int ticket = 0;
      if (lane == 0) ticket = atomicAdd(&a.tickets[tile], 1u);
      ticket = __shfl_sync(0xFFFFFFFFu, ticket, 0);
      const bool last = ticket == static_cast<unsigned int>(a.k_slices - 1);   // else another warp finishes this tile
      if (last) {
      __threadfence();
      acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
      for (int sl = 0; sl < a.k_slices; ++sl) {                            // fixed order: deterministic sum
        const float* p = a.partial + (static_cast<size_t>(sl) * a.tiles + tile) * 128;
        const float2 lo2 = __ldcg(reinterpret_cast<const float2*>(p + g * 8 + col));
        const float2 hi2 = __ldcg(reinterpret_cast<const float2*>(p + (g + 8) * 8 + col));
        acc[0] += lo2.x; acc[1] += lo2.y; acc[2] += hi2.x; acc[3] += hi2.y;
      }
      if (lane == 0) a.tickets[tile] = 0;                                  // ready for the next call
      }
      write_out = last;
    }
    if (write_out && row_a < a.n) {
      if (col < a.m) a.y[static_cast<size_t>(col) * a.ldy + row_a] = __float2bfloat16_rn(acc[0]);
      if (col + 1 < a.m) a.y[static_cast<size_t>(col + 1) * a.ldy + row_a] = __float2bfloat16_rn(acc[1]);
    }
    if (write_out && row_b < a.n) {
      if (col < a.m) a.y[static_cast<size_t>(col) * a.ldy + row_b] = __float2bfloat16_rn(acc[2]);
      if (col + 1 < a.m) a.y[static_cast<size_t>(col + 1) * a.ldy + row_b] = __float2bfloat16_rn(acc[3]);
    }
    q += kGemvWarps / kGemvParts;
    __syncwarp();                        // every lane is done with the ring before the next tile refills it
    have_tile = open_tile(q);
    if (have_tile) prime();
  }
}

// Workspace layout: uint32 tickets, then [8][tiles][16][8] float32 partial sums.  The ticket area is sized
// from the workspace's capacity, not from this call's n, so that calls with different n that share a
// workspace never see another call's partial sums where they expect zeroed tickets.
static int64_t gemv_ws_bytes_for_tiles(int64_t tiles) { return ((tiles * 4 + 255) / 256) * 256 + 8 * tiles * 128 * 4; }
static int64_t gemv_ws_bytes(int64_t n) { return gemv_ws_bytes_for_tiles((n + 15) / 16); }
// largest number of 16-row tiles a workspace of `bytes` can serve
static int64_t gemv_ws_capacity(int64_t bytes) {
  int64_t t = bytes / (4 + 8 * 128 * 4);
  while (t > 0 && gemv_ws_bytes_for_tiles(t) > bytes) --t;
  return t;
}

template <int D>
static int launch_gemv(const GemvArgs& a, int grid, size_t smem, cudaStream_t stream) {
  static thread_local int attr_dev = -1;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    PLQ_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_dev = dev;
  }
  gemv_kernel<D><<<grid, kGemvThreads, smem, stream>>>(a);
  PLQ_CUDA_TRY(cudaGetLastError());
  return PLQ_OK;
}

// Argument and device checks shared by the two GEMV entry points; nothing is launched or touched before they pass.
static int check_gemv_args(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                           const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                           int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, const void* y_bf16, int64_t ldy) {
  if (m < 1 || m > 8 || n < 1 || k_lo < 0 || k_hi < 0 || k_lo + k_hi <= 0 || ldy < n) return PLQ_ERR_SHAPE;
  if (k_lo % 64 != 0 || k_hi % 32 != 0) return PLQ_ERR_SHAPE;
  if (k_lo + k_hi > 32768 * 8 || n > (1 << 30)) return PLQ_ERR_LIMIT;
  if (!y_bf16) return PLQ_ERR_NULL;
  if (k_lo && (!a_lo_codes || !a_lo_sf || !b_lo_codes || !b_lo_sf)) return PLQ_ERR_NULL;
  if (k_hi && (!a_hi_codes || !a_hi_sf || !b_hi_codes || !b_hi_sf)) return PLQ_ERR_NULL;
  if (!aligned16(a_lo_codes) || !aligned16(b_lo_codes) || !aligned16(a_hi_codes) || !aligned16(b_hi_codes) ||
      !aligned16(a_lo_sf) || !aligned16(b_lo_sf))
    return PLQ_ERR_ALIGN;
  return device_check();
}

}  // namespace plq

extern "C" int64_t plq_gemv_workspace_bytes(int64_t n) { return n > 0 ? plq::gemv_ws_bytes(n) : 0; }

extern "C" int plq_gemv(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                        const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                        int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy,
                        void* workspace, int64_t workspace_bytes, void* stream) {
  using namespace plq;
  int st = check_gemv_args(a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf, m, n, k_lo,
                           k_hi, y_bf16, ldy);
  if (st != PLQ_OK) return st;
  if (!aligned16(workspace)) return PLQ_ERR_ALIGN;

  GemvArgs a;
  a.a_lo = static_cast<const uint8_t*>(a_lo_codes); a.a_lo_sf = static_cast<const uint8_t*>(a_lo_sf);
  a.a_hi = static_cast<const uint8_t*>(a_hi_codes); a.a_hi_sf = static_cast<const uint8_t*>(a_hi_sf);
  a.b_lo = static_cast<const uint8_t*>(b_lo_codes); a.b_lo_sf = static_cast<const uint8_t*>(b_lo_sf);
  a.b_hi = static_cast<const uint8_t*>(b_hi_codes); a.b_hi_sf = static_cast<const uint8_t*>(b_hi_sf);
  a.m = static_cast<int>(m); a.n = static_cast<int>(n);
  a.k_lo = static_cast<int>(k_lo); a.k_hi = static_cast<int>(k_hi);
  a.y = static_cast<__nv_bfloat16*>(y_bf16); a.ldy = ldy;
  a.tiles = static_cast<int>((n + 15) / 16);

  // K slices: enough (tile, slice) units to give every SM about one per warp, and a slice of the
  // activations small enough for shared memory.  Without a workspace only one slice is possible.
  const int sms = sm_count();
  const int chunks = static_cast<int>((k_lo + 127) / 128);
  const int hblocks = static_cast<int>(k_hi / 32);
  const bool have_ws = workspace != nullptr && workspace_bytes >= gemv_ws_bytes(n);
  const int64_t tiles_cap = have_ws ? gemv_ws_capacity(workspace_bytes) : 0;
  const int64_t ticket_bytes = ((tiles_cap * 4 + 255) / 256) * 256;
  int ks = 1;
  while (ks < 8 && have_ws && ((chunks + ks - 1) / ks > 32 || static_cast<int64_t>(a.tiles) * ks < 10LL * sms) &&
         chunks >= 4 * ks)
    ks *= 2;
  a.k_slices = ks;
  a.cps = (chunks + ks - 1) / ks;
  a.hps = (hblocks + ks - 1) / ks;
  const size_t x_bytes = static_cast<size_t>(a.cps) * 2048 + static_cast<size_t>(a.hps) * (512 + 32);
  const size_t budget = 226 * 1024 - kGemvRedBytes;
  if (x_bytes + 2 * kGemvWarps * kRingStageBytes > budget) return have_ws ? PLQ_ERR_LIMIT : PLQ_ERR_NULL;
  const int d_fit = static_cast<int>((budget - x_bytes) / (kGemvWarps * kRingStageBytes));
  const int depth = d_fit >= 8 ? 8 : (d_fit >= 4 ? 4 : 2);
  const size_t smem = x_bytes + static_cast<size_t>(depth) * kGemvWarps * kRingStageBytes + kGemvRedBytes;
  a.tickets = static_cast<unsigned int*>(workspace);
  a.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ticket_bytes);
  const int64_t units = static_cast<int64_t>(a.tiles) * ks;
  const int grid = static_cast<int>(units < sms ? units : sms);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (depth == 8) return launch_gemv<8>(a, grid, smem, s);
  if (depth == 4) return launch_gemv<4>(a, grid, smem, s);
  return launch_gemv<2>(a, grid, smem, s);
}

// ---- decode GEMV for callers that cannot provide scratch memory ---------------------------------
//
// Some hosts of this library have no way to hand it a workspace: an inference server that reserved
// all of HBM for its own pool at start-up (a later cudaMalloc simply fails), or a plugin that sits
// behind an interface which passes inputs and outputs only and has no handle to the host's
// allocator.  For them the K-slice scratch of the GEMV lives in the library image itself: a
// file-scope device array, present on every GPU that loads the library until the process exits.
namespace plq {
constexpr int64_t kGemvStaticMaxRows = 32768;                         // largest n the built-in scratch serves
constexpr int64_t kGemvStaticBytes = ((kGemvStaticMaxRows / 16 * 4 + 255) / 256) * 256 + 8 * (kGemvStaticMaxRows / 16) * 128 * 4;
static __device__ __align__(256) unsigned char g_gemv_scratch[kGemvStaticBytes];   // ~8.4 MB; zero at load

// In host code `g_gemv_scratch` is only a handle for the runtime, not an address a kernel can use:
// the device address is looked up once per device, with that device current, and published atomically
// (two host threads that both make the first call on a device resolve the same address).
static std::atomic<void*> g_gemv_scratch_ptr[64];
}  // namespace plq

extern "C" int plq_gemv_static_scratch(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes,
                                       const void* a_hi_sf, const void* b_lo_codes, const void* b_lo_sf,
                                       const void* b_hi_codes, const void* b_hi_sf, int64_t m, int64_t n,
                                       int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy, void* stream) {
  using namespace plq;
  // every check first (shapes, pointers, device): a rejected call touches nothing
  const int st = check_gemv_args(a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf, m, n,
                                 k_lo, k_hi, y_bf16, ldy);
  if (n > kGemvStaticMaxRows) return PLQ_ERR_LIMIT;    // built-in scratch covers n <= 32768 only
  if (st != PLQ_OK) return st;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return PLQ_ERR_LIMIT;
  void* ptr = g_gemv_scratch_ptr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // first call on this device: resolve the array's device address and make sure the tickets start at
    // zero (they do at load; the kernel leaves them zero after every call)
    PLQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_gemv_scratch));
    PLQ_CUDA_TRY(cudaMemsetAsync(ptr, 0, ((gemv_ws_capacity(kGemvStaticBytes) * 4 + 255) / 256) * 256,
                                 static_cast<cudaStream_t>(stream)));
    g_gemv_scratch_ptr[dev].store(ptr, std::memory_order_release);
  }
  return plq_gemv(a_lo_codes, a_lo_sf, a_hi_codes, a_hi_sf, b_lo_codes, b_lo_sf, b_hi_codes, b_hi_sf, m, n, k_lo, k_hi,
                  y_bf16, ldy, ptr, kGemvStaticBytes, stream);
}
