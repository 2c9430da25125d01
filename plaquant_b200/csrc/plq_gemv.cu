// Decode GEMV for m <= 8 tokens: y[m, n] = deq(A)[m, :] . deq(B)[n, :], HBM-bound on B.
//
// The weights are streamed exactly once with 16-byte loads; each warp owns 16 weight rows and
// uses the warp-level m16n8k16 f16 MMA as its dot-product engine (A fragment = 16 weight rows,
// B fragment = the <= 8 activation rows), because eight tokens times ~7 CUDA-core operations
// per weight element would not keep up with HBM.  Products are exact in f16 (E2M1 x E4M3 and
// E4M3 values are f16-representable), accumulation is float32.
//
//   * Lane (g = lane / 4, t = lane % 4) loads, per 128-element K chunk, the 16 bytes that hold
//     elements 32t .. 32t+31 of rows g and g+8.  The MMA sums over K, so which K elements sit
//     in which fragment slot is free as long as both operands agree: MMA number j of a chunk
//     consumes elements 32t + 4j .. 32t + 4j + 3 of every lane.  No cross-lane shuffle of weight data.
//   * The activation slice is dequantised once per CTA into shared memory, already arranged in
//     B-fragment order, so the inner loop reads it with conflict-free 16-byte loads.
//   * NVFP4 scales are folded into the f16 operands (exact); MXFP8 scales are powers of two
//     applied in float32 after the two MMAs of a 32-element block.
//   * K is cut into slices, one CTA of a thread-block cluster each; partial sums are combined
//     through distributed shared memory in rank order, so results are deterministic.
#include <cooperative_groups.h>

#include "plq_quant.cuh"

namespace cg = cooperative_groups;

namespace plq {

struct GemvArgs {
  const uint8_t *a_lo, *a_lo_sf, *a_hi, *a_hi_sf;   // activations, m rows, row-major scales
  const uint8_t *b_lo, *b_lo_sf, *b_hi, *b_hi_sf;   // weights, n rows, row-major scales
  int m, n, k_lo, k_hi;
  __nv_bfloat16* y;
  int64_t ldy;
  int k_slices, cps, hps;   // lo chunks (128 elements) and hi blocks (32 elements) per slice
};

constexpr int kGemvThreads = 256;
constexpr int kGemvRowsPerCta = 128;
constexpr int kGemvUnroll = 4;

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

__global__ void __launch_bounds__(kGemvThreads) gemv_kernel(const GemvArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint4* xs_lo = reinterpret_cast<uint4*>(smem);                          // [cps][4][32] x 8 f16
  uint4* xs_hi = xs_lo + a.cps * 128;                                      // [hps][32] x 8 f16
  float* sxh = reinterpret_cast<float*>(xs_hi + a.hps * 32);               // [hps][8]
  float* part = sxh + a.hps * 8;                                           // [128][8]

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int slice = blockIdx.y;
  const int n0 = blockIdx.x * kGemvRowsPerCta;

  const int total_chunks = (a.k_lo + 127) >> 7;
  const int c_begin = min(slice * a.cps, total_chunks);
  const int c_end = min(c_begin + a.cps, total_chunks);
  const int total_hb = a.k_hi >> 5;
  const int h_begin = min(slice * a.hps, total_hb);
  const int h_end = min(h_begin + a.hps, total_hb);

  // ---- stage the activation slice, dequantised, in fragment order -------------------------
  {
    const int units = (c_end - c_begin) * 16;           // 8-element units per row in this slice
    for (int it = tid; it < units * 8; it += kGemvThreads) {
      const int row = it / units, u = it % units;
      const int c = u >> 4, tt = (u >> 2) & 3, jj = u & 3;
      const int k = (c_begin + c) * 128 + tt * 32 + jj * 8;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (row < a.m && k < a.k_lo) {
        const uint32_t codes = *reinterpret_cast<const uint32_t*>(a.a_lo + (static_cast<size_t>(row) * a.k_lo + k) / 2);
        const uint32_t sc = a.a_lo_sf[static_cast<size_t>(row) * (a.k_lo >> 4) + (k >> 4)];
        uint32_t s2 = cvt_e4m3x2_to_f16x2(sc | (sc << 8));
        cvt_e2m1x8_to_f16x2(codes, o.x, o.y, o.z, o.w);
        o.x = hmul2_u32(o.x, s2); o.y = hmul2_u32(o.y, s2);
        o.z = hmul2_u32(o.z, s2); o.w = hmul2_u32(o.w, s2);
      }
      xs_lo[(c * 4 + jj) * 32 + row * 4 + tt] = o;
    }
    const int hunits = (h_end - h_begin) * 4;
    for (int it = tid; it < hunits * 8; it += kGemvThreads) {
      const int row = it / hunits, u = it % hunits;
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

  // ---- stream the weights ---------------------------------------------------------------
  const int row_a = n0 + warp * 16 + g, row_b = row_a + 8;
  const int ra = min(row_a, a.n - 1), rb = min(row_b, a.n - 1);
  const uint8_t* wa = a.b_lo + static_cast<size_t>(ra) * (a.k_lo >> 1) + t * 16;
  const uint8_t* wb = a.b_lo + static_cast<size_t>(rb) * (a.k_lo >> 1) + t * 16;
  const uint8_t* sa = a.b_lo_sf + static_cast<size_t>(ra) * (a.k_lo >> 4) + t * 2;
  const uint8_t* sb = a.b_lo_sf + static_cast<size_t>(rb) * (a.k_lo >> 4) + t * 2;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};

  for (int c0 = c_begin; c0 < c_end; c0 += kGemvUnroll) {
    uint4 va[kGemvUnroll], vb[kGemvUnroll];
    uint32_t fa[kGemvUnroll], fb[kGemvUnroll];
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int c = c0 + u;
      const bool ok = c < c_end && (c * 128 + t * 32) < a.k_lo;
      va[u] = vb[u] = make_uint4(0, 0, 0, 0);
      fa[u] = fb[u] = 0;
      if (ok) {
        va[u] = __ldcs(reinterpret_cast<const uint4*>(wa + c * 64));
        vb[u] = __ldcs(reinterpret_cast<const uint4*>(wb + c * 64));
        fa[u] = *reinterpret_cast<const uint16_t*>(sa + c * 8);
        fb[u] = *reinterpret_cast<const uint16_t*>(sb + c * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < kGemvUnroll; ++u) {
      const int c = c0 + u;
      if (c >= c_end) break;
      const uint32_t sfa = cvt_e4m3x2_to_f16x2(fa[u]), sfb = cvt_e4m3x2_to_f16x2(fb[u]);
      const uint32_t sa0 = __byte_perm(sfa, sfa, 0x1010), sa1 = __byte_perm(sfa, sfa, 0x3232);
      const uint32_t sb0 = __byte_perm(sfb, sfb, 0x1010), sb1 = __byte_perm(sfb, sfb, 0x3232);
      const uint32_t wva[4] = {va[u].x, va[u].y, va[u].z, va[u].w};
      const uint32_t wvb[4] = {vb[u].x, vb[u].y, vb[u].z, vb[u].w};
      const uint4* xrow = xs_lo + (c - c_begin) * 128 + lane;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const uint4 xb = xrow[jj * 32];
        const uint32_t scale_a = jj < 2 ? sa0 : sa1, scale_b = jj < 2 ? sb0 : sb1;
        uint32_t a0, a1, a2, a3, e0, e1, e2, e3;
        cvt_e2m1x8_to_f16x2(wva[jj], a0, a2, e0, e2);
        cvt_e2m1x8_to_f16x2(wvb[jj], a1, a3, e1, e3);
        mma_16816(acc, hmul2_u32(a0, scale_a), hmul2_u32(a1, scale_b), hmul2_u32(a2, scale_a),
                  hmul2_u32(a3, scale_b), xb.x, xb.y);
        mma_16816(acc, hmul2_u32(e0, scale_a), hmul2_u32(e1, scale_b), hmul2_u32(e2, scale_a),
                  hmul2_u32(e3, scale_b), xb.z, xb.w);
      }
    }
  }

  // ---- MXFP8 outlier columns ----------------------------------------------------------------
  for (int hb = h_begin; hb < h_end; ++hb) {
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

  // ---- combine the K slices and store ---------------------------------------------------------
  if (a.k_slices == 1) {
    const int col = 2 * t;
    if (row_a < a.n) {
      if (col < a.m) a.y[static_cast<size_t>(col) * a.ldy + row_a] = __float2bfloat16_rn(acc[0]);
      if (col + 1 < a.m) a.y[static_cast<size_t>(col + 1) * a.ldy + row_a] = __float2bfloat16_rn(acc[1]);
    }
    if (row_b < a.n) {
      if (col < a.m) a.y[static_cast<size_t>(col) * a.ldy + row_b] = __float2bfloat16_rn(acc[2]);
      if (col + 1 < a.m) a.y[static_cast<size_t>(col + 1) * a.ldy + row_b] = __float2bfloat16_rn(acc[3]);
    }
    return;
  }
  cg::cluster_group cluster = cg::this_cluster();
  {
    const int r = warp * 16 + g;
    part[r * 8 + 2 * t] = acc[0];
    part[r * 8 + 2 * t + 1] = acc[1];
    part[(r + 8) * 8 + 2 * t] = acc[2];
    part[(r + 8) * 8 + 2 * t + 1] = acc[3];
  }
  cluster.sync();
  {
    const int rank = static_cast<int>(cluster.block_rank());
    const int rows_per_rank = kGemvRowsPerCta / a.k_slices;
    for (int o = tid; o < rows_per_rank * 8; o += kGemvThreads) {
      const int r = rank * rows_per_rank + (o >> 3), col = o & 7;
      float s = 0.0f;
      for (int rr = 0; rr < a.k_slices; ++rr) s += cluster.map_shared_rank(part, rr)[r * 8 + col];
      if (col < a.m && n0 + r < a.n) a.y[static_cast<size_t>(col) * a.ldy + n0 + r] = __float2bfloat16_rn(s);
    }
  }
  cluster.sync();   // keep every CTA's shared memory alive until all ranks have read it
}

}  // namespace plq

extern "C" int plq_gemv(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                        const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                        int64_t m, int64_t n, int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy,
                        void* stream) {
  using namespace plq;
  if (m < 1 || m > 8 || n < 1 || k_lo < 0 || k_hi < 0 || k_lo + k_hi <= 0 || ldy < n) return PLQ_ERR_SHAPE;
  if (k_lo % 64 != 0 || k_hi % 32 != 0) return PLQ_ERR_SHAPE;
  if (k_lo + k_hi > 32768 * 8 || n > (1 << 30)) return PLQ_ERR_LIMIT;
  if (!y_bf16) return PLQ_ERR_NULL;
  if (k_lo && (!a_lo_codes || !a_lo_sf || !b_lo_codes || !b_lo_sf)) return PLQ_ERR_NULL;
  if (k_hi && (!a_hi_codes || !a_hi_sf || !b_hi_codes || !b_hi_sf)) return PLQ_ERR_NULL;
  if (!aligned16(a_lo_codes) || !aligned16(b_lo_codes) || !aligned16(a_hi_codes) || !aligned16(b_hi_codes) ||
      !aligned16(a_lo_sf) || !aligned16(b_lo_sf))
    return PLQ_ERR_ALIGN;
  int st = device_check();
  if (st != PLQ_OK) return st;

  GemvArgs a;
  a.a_lo = static_cast<const uint8_t*>(a_lo_codes); a.a_lo_sf = static_cast<const uint8_t*>(a_lo_sf);
  a.a_hi = static_cast<const uint8_t*>(a_hi_codes); a.a_hi_sf = static_cast<const uint8_t*>(a_hi_sf);
  a.b_lo = static_cast<const uint8_t*>(b_lo_codes); a.b_lo_sf = static_cast<const uint8_t*>(b_lo_sf);
  a.b_hi = static_cast<const uint8_t*>(b_hi_codes); a.b_hi_sf = static_cast<const uint8_t*>(b_hi_sf);
  a.m = static_cast<int>(m); a.n = static_cast<int>(n);
  a.k_lo = static_cast<int>(k_lo); a.k_hi = static_cast<int>(k_hi);
  a.y = static_cast<__nv_bfloat16*>(y_bf16); a.ldy = ldy;

  const int n_blocks = static_cast<int>((n + kGemvRowsPerCta - 1) / kGemvRowsPerCta);
  const int chunks = static_cast<int>((k_lo + 127) / 128);
  const int hblocks = static_cast<int>(k_hi / 32);
  int ks = 1;
  const int target = 2 * sm_count();
  while (ks < 8 && (n_blocks * ks < target || (chunks + ks - 1) / ks > 32) && chunks / (2 * ks) >= 2) ks *= 2;
  a.k_slices = ks;
  a.cps = (chunks + ks - 1) / ks;
  a.hps = (hblocks + ks - 1) / ks;
  if (a.cps > 48) return PLQ_ERR_LIMIT;
  const size_t smem = static_cast<size_t>(a.cps) * 2048 + static_cast<size_t>(a.hps) * (512 + 32) + 4096;

  static thread_local int attr_done_dev = -1;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_done_dev != dev) {
    PLQ_CUDA_TRY(cudaFuncSetAttribute(gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
    attr_done_dev = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_blocks), static_cast<unsigned>(ks), 1);
  cfg.blockDim = dim3(kGemvThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = static_cast<unsigned>(ks);
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  PLQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_kernel, a));
  return PLQ_OK;
}
