// Quantise-and-pack kernels: [RMSNorm] -> [block-Hadamard 128] -> NVFP4 | MXFP8 codes + scales,
// and the inverse (dequantise to bf16).  HBM-bound elementwise work, one CTA per row.
//
// Thread mapping.  A row is cut into 128-element blocks (the Hadamard block).  Four
// consecutive lanes (a "quad", q = lane & 3) own one block; lane q holds the 32 elements
// e = 32*j + 8*q + i (j = 0..3, i = 0..7), i.e. four 16-byte loads, so every 32-byte sector
// fetched from HBM is consumed whole.  In this mapping
//   * butterfly strides 1,2,4 (bits of i) and 32,64 (bits of j) stay inside a lane,
//     strides 8,16 (bits of q) are two shuffle rounds inside the quad;
//   * an NVFP4 block (16 elements) is one j of lanes {0,1} or {2,3}: one shuffle for the max;
//   * an MXFP8 block (32 elements) is one j of the whole quad: two shuffles;
//   * the NVFP4/MXFP8 boundary (a multiple of 64) never cuts a j group.
// Summation and butterfly order are fixed and documented in the CPU oracle
// (`_sumsq_det`, `block_hadamard_det`), which these kernels match bit for bit.
#include "plq_quant.cuh"

namespace plq {

struct PackArgs {
  const uint4* x;        // bf16 [rows, k], row stride ldx8 * 8 elements
  const uint4* x2;       // prologue 1: the "up" half, same stride as x; prologue 2: the residual [rows, k], contiguous
  uint4* h_out;          // prologue 2: bf16 [rows, k], receives residual + x
  int ldx8;              // row stride of x (and of x2 in prologue 1) in 16-byte units
  // prologue 3 (tensor-parallel): x = sum over the ranks of their [rows, k] buffers, read over NVLink
  const uint4* const* peer_x;    // device array [world] of buffer addresses (this rank's own included)
  int* const* peer_flags;        // device array [world]: rank r's int32 flags[world]
  int* flags;                    // this rank's flags[world]: flags[r] = last call rank r has announced
  int* sync;                     // this rank's {calls completed, CTAs finished in the current call}
  int32_t* status;               // receives PLQ_DEV_TIMEOUT if a rank does not show up
  int world, rank;
  const uint4* gamma;    // bf16 [k] (RMSNorm weight) or nullptr
  float eps;
  int rows, k, k_lo;     // k_hi = k - k_lo
  uint8_t* lo_codes;     // [rows, k_lo/2]
  uint8_t* lo_sf;
  uint8_t* hi_codes;     // [rows, k_hi]
  uint8_t* hi_sf;
  int sf_tiled;
  int lo_chunks, hi_chunks;  // chunks per 128-row group in the tiled layouts
};

// PRO selects what is quantised: 0 = x; 1 = SiLU(x) * x2 (gate and up halves of the MLP, rounded to bf16 after
// the activation and after the product like the two PyTorch ops they replace, inference/forward_pass.py:266
// in the reference); 2 = x2 + x (residual add, one rounding, also written to h_out: forward_pass.py:258-262);
// 3 = like 2 with x = bf16(sum over the tensor-parallel ranks of their partial outputs), float32 sum in rank order,
// read from the peers' memory: the all-reduce after a row-parallel linear, the residual add, the norm and the
// quantiser of the next linear in one kernel.
template <int PRO, bool NORM, bool HAD>
__global__ void __launch_bounds__(1024) pack_kernel(const PackArgs a) {
  // Programmatic dependent launch on both sides.  A consumer launched with programmatic stream serialisation
  // (GEMM, decode GEMV) may set itself up and prefetch its weights while this kernel runs; it waits for this
  // grid's completion before reading the codes.  This kernel itself may be launched before its predecessor
  // has finished, and waits here before it reads anything.
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int q = tid & 3;
  const int k0 = (tid >> 2) * 128;                  // first element of this quad's block
  const int lane = tid & 31;
  if constexpr (PRO == 3) {
    // Cross-rank handshake.  Call number c = completed calls + 1.  This rank's partial output was written by
    // the preceding kernel of the stream; block 0 announces it by storing c into flags[rank] of every peer, and
    // every block waits (bounded) until all peers have announced c in this rank's flags.  Buffers alternate
    // between two per call site order, so a peer that runs ahead never overwrites what is being read here.
    const int call = *reinterpret_cast<volatile int*>(a.sync) + 1;
    if (blockIdx.x == 0 && tid < a.world) {
      __threadfence_system();
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[tid] + a.rank), "r"(call) : "memory");
    }
    if (tid < a.world) {
      const long long t0 = clock64();
      int seen;
      do {
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(a.flags + tid) : "memory");
        if (seen - call >= 0) break;
        if (clock64() - t0 > kWaitLimitCycles) {        // a rank is missing: report and go on (the result is void)
          atomicExch(a.status, PLQ_DEV_TIMEOUT);
          break;
        }
      } while (true);
    }
    __syncthreads();
  }
  // v2[p] holds elements (2p, 2p+1) of the lane's 32, i.e. e = 8*j + i -> p = 4*j + i/2.  Arithmetic on
  // pairs uses the packed float32x2 instructions of sm_100 (same IEEE rounding per element, half the issue slots).
  float2 v2[16];

  // ---- load: four 16-byte pieces per lane ---------------------------------------------
  const uint4* xrow = a.x + static_cast<size_t>(row) * a.ldx8;
  uint4 wsum[PRO == 3 ? 4 : 1];
  if constexpr (PRO == 3) {
    // x = bf16(sum over the ranks), float32 in rank order (every rank computes the same bits).  The peer loads
    // of two of the lane's four pieces are all issued before any of them is used: two NVLink round trips per
    // lane instead of one per rank and piece.
#pragma unroll
    for (int jp = 0; jp < 4; jp += 2) {
      uint4 t[2][8];
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int kk = k0 + 32 * (jp + jj) + 8 * q;
        const size_t off = static_cast<size_t>(row) * (a.k >> 3) + (kk >> 3);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          t[jj][r] = make_uint4(0, 0, 0, 0);
          if (r < a.world && kk < a.k)
            asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(t[jj][r].x), "=r"(t[jj][r].y), "=r"(t[jj][r].z), "=r"(t[jj][r].w)
                         : "l"(a.peer_x[r] + off)
                         : "memory");
        }
      }
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < a.world) {
            const uint32_t tt[4] = {t[jj][r].x, t[jj][r].y, t[jj][r].z, t[jj][r].w};
#pragma unroll
            for (int p = 0; p < 4; ++p)
              acc[p] = __fadd2_rn(acc[p], make_float2(bf16lo_to_f32(tt[p]), bf16hi_to_f32(tt[p])));
          }
        }
        wsum[jp + jj] = make_uint4(f32x2_to_bf16x2(acc[0].x, acc[0].y), f32x2_to_bf16x2(acc[1].x, acc[1].y),
                                   f32x2_to_bf16x2(acc[2].x, acc[2].y), f32x2_to_bf16x2(acc[3].x, acc[3].y));
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int kk = k0 + 32 * j + 8 * q;
    uint4 w = make_uint4(0, 0, 0, 0);
    if constexpr (PRO == 3) {
      w = wsum[j];
    } else {
      if (kk < a.k) w = __ldg(xrow + (kk >> 3));
    }
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    if constexpr (PRO == 0) {
#pragma unroll
      for (int p = 0; p < 4; ++p) v2[4 * j + p] = make_float2(bf16lo_to_f32(ww[p]), bf16hi_to_f32(ww[p]));
    } else if constexpr (PRO == 1) {
      uint4 u = make_uint4(0, 0, 0, 0);
      if (kk < a.k) u = __ldg(a.x2 + static_cast<size_t>(row) * a.ldx8 + (kk >> 3));
      const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float g0 = bf16lo_to_f32(ww[p]), g1 = bf16hi_to_f32(ww[p]);
        const uint32_t t = f32x2_to_bf16x2(g0 / (1.0f + expf(-g0)), g1 / (1.0f + expf(-g1)));   // SiLU, to bf16
        const float2 prod = __fmul2_rn(make_float2(bf16lo_to_f32(t), bf16hi_to_f32(t)),
                                       make_float2(bf16lo_to_f32(uu[p]), bf16hi_to_f32(uu[p])));
        const uint32_t b = f32x2_to_bf16x2(prod.x, prod.y);                                       // product, to bf16
        v2[4 * j + p] = make_float2(bf16lo_to_f32(b), bf16hi_to_f32(b));
      }
    } else {
      uint4 r = make_uint4(0, 0, 0, 0);
      if (kk < a.k) r = __ldg(a.x2 + static_cast<size_t>(row) * (a.k >> 3) + (kk >> 3));
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
      uint32_t hh[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 sum = __fadd2_rn(make_float2(bf16lo_to_f32(rr[p]), bf16hi_to_f32(rr[p])),
                                      make_float2(bf16lo_to_f32(ww[p]), bf16hi_to_f32(ww[p])));
        hh[p] = f32x2_to_bf16x2(sum.x, sum.y);
        v2[4 * j + p] = make_float2(bf16lo_to_f32(hh[p]), bf16hi_to_f32(hh[p]));
      }
      if (kk < a.k) a.h_out[static_cast<size_t>(row) * (a.k >> 3) + (kk >> 3)] = make_uint4(hh[0], hh[1], hh[2], hh[3]);
    }
  }

  // ---- RMSNorm (inference/forward_pass.py:33-39 in the reference) ------------------------
  if constexpr (NORM) {
    __shared__ float warp_sums[32];
    uint4 gpre[4];                                      // the norm weights: requested now, needed after the row sum
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kk = k0 + 32 * j + 8 * q;
      gpre[j] = make_uint4(0, 0, 0, 0);
      if (kk < a.k) gpre[j] = __ldg(a.gamma + (kk >> 3));
    }
    float2 s2 = make_float2(0.0f, 0.0f);               // even and odd elements accumulate separately
#pragma unroll
    for (int p = 0; p < 16; ++p) s2 = __ffma2_rn(v2[p], v2[p], s2);   // v*v is exact for bf16 inputs
    float s = __fadd_rn(s2.x, s2.y);
    s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 1);
    s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 2);              // (p0+p1)+(p2+p3): block sum
    s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 4);
    s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 8);
    s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 16);             // eight blocks, pairwise tree
    if (lane == 0) warp_sums[tid >> 5] = s;
    __syncthreads();
    float tot = 0.0f;
    const int nwarps = blockDim.x >> 5;
    for (int w = 0; w < nwarps; ++w) tot = tot + warp_sums[w];  // left to right
    const float var = __fdiv_rn(tot, static_cast<float>(a.k));
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
    const float2 r2 = make_float2(r, r);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t gw[4] = {gpre[j].x, gpre[j].y, gpre[j].z, gpre[j].w};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const float2 y = __fmul2_rn(make_float2(bf16lo_to_f32(gw[p]), bf16hi_to_f32(gw[p])), __fmul2_rn(v2[4 * j + p], r2));
        const uint32_t b = f32x2_to_bf16x2(y.x, y.y);
        v2[4 * j + p] = make_float2(bf16lo_to_f32(b), bf16hi_to_f32(b));
      }
    }
  }

  // ---- block-Hadamard(128): strides 1,2,4 | 8,16 (shuffles) | 32,64, then * 1/sqrt(128) ----
  if constexpr (HAD) {
    const float2 neg1 = make_float2(-1.0f, -1.0f);
#pragma unroll
    for (int p = 0; p < 16; ++p) {                       // stride 1: inside a pair
      const float x0 = v2[p].x, x1 = v2[p].y;
      v2[p] = make_float2(__fadd_rn(x0, x1), __fsub_rn(x0, x1));
    }
#pragma unroll
    for (int h = 1; h < 4; h <<= 1) {                    // strides 2, 4: pairs p, p + h
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        if ((p & h) == 0) {
          const float2 x0 = v2[p], x1 = v2[p + h];
          v2[p] = __fadd2_rn(x0, x1);
          v2[p + h] = __ffma2_rn(x1, neg1, x0);          // x0 - x1: exact product, one rounding
        }
      }
    }
#pragma unroll
    for (int m = 1; m <= 2; m <<= 1) {                   // strides 8, 16: across the quad
      const float sg = (q & m) ? -1.0f : 1.0f;           // upper lane of the pair computes partner - own
      const float2 sgn = make_float2(sg, sg);
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        float2 o;
        o.x = __shfl_xor_sync(0xFFFFFFFFu, v2[p].x, m);
        o.y = __shfl_xor_sync(0xFFFFFFFFu, v2[p].y, m);
        v2[p] = __ffma2_rn(sgn, v2[p], o);               // own + other / other - own
      }
    }
#pragma unroll
    for (int h = 4; h < 16; h <<= 1) {                   // strides 32, 64: pairs p, p + h
#pragma unroll
      for (int p = 0; p < 16; ++p) {
        if ((p & h) == 0) {
          const float2 x0 = v2[p], x1 = v2[p + h];
          v2[p] = __fadd2_rn(x0, x1);
          v2[p + h] = __ffma2_rn(x1, neg1, x0);
        }
      }
    }
    const float2 scale = make_float2(0.088388347648318441f, 0.088388347648318441f);
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      const float2 y = __fmul2_rn(v2[p], scale);
      const uint32_t b = f32x2_to_bf16x2(y.x, y.y);
      v2[p] = make_float2(bf16lo_to_f32(b), bf16hi_to_f32(b));
    }
  }

  // ---- quantise, 32 elements (one j group of the quad) at a time ---------------------------
  uint32_t lo_sf_bytes = 0;                           // this lane pair's scale byte for j = 0..3
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int kg = k0 + 32 * j;                       // first element of the quad's j group
    float x8[8];
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x8[2 * i] = v2[4 * j + i].x;
      x8[2 * i + 1] = v2[4 * j + i].y;
      m = fmaxf(m, fmaxf(fabsf(x8[2 * i]), fabsf(x8[2 * i + 1])));
    }
    m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    const float m32 = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    if (kg >= a.k) continue;
    if (kg < a.k_lo) {
      const uint32_t c = nvfp4_scale_code(m);
      const float s = e4m3_code_to_f32(c);
      const uint32_t codes = nvfp4_quantize8(x8, s, __frcp_rn(s));
      *reinterpret_cast<uint32_t*>(a.lo_codes + (static_cast<size_t>(row) * a.k_lo + kg + 8 * q) / 2) = codes;
      lo_sf_bytes |= c << (8 * j);
    } else {
      const uint32_t c = mxfp8_scale_code(m32);
      const uint2 codes = mxfp8_quantize8(x8, __uint_as_float((254u - c) << 23));
      const int kh = kg - a.k_lo;
      *reinterpret_cast<uint2*>(a.hi_codes + static_cast<size_t>(row) * (a.k - a.k_lo) + kh + 8 * q) = codes;
      if (q == 0) {
        const int kb = kh >> 5;
        const size_t off = a.sf_tiled ? static_cast<size_t>(sf_tiled_offset(row, kb, a.hi_chunks))
                                      : static_cast<size_t>(row) * ((a.k - a.k_lo) >> 5) + kb;
        a.hi_sf[off] = static_cast<uint8_t>(c);
      }
    }
  }
  // NVFP4 scales: lanes 0/1 of the quad hold blocks 0,2,4,6 (one byte per j), lanes 2/3 hold
  // blocks 1,3,5,7.  Lane 0 interleaves them into two 4-byte words (64 elements each).
  const uint32_t odd = __shfl_xor_sync(0xFFFFFFFFu, lo_sf_bytes, 2);
  if (q == 0) {
    const uint32_t w0 = __byte_perm(lo_sf_bytes, odd, 0x5140);   // blocks 0,1,2,3
    const uint32_t w1 = __byte_perm(lo_sf_bytes, odd, 0x7362);   // blocks 4,5,6,7
    const int kb = k0 >> 4;                                      // first 16-block index of this quad
    if (a.sf_tiled) {
      if (k0 < a.k_lo) *reinterpret_cast<uint32_t*>(a.lo_sf + sf_tiled_offset(row, kb, a.lo_chunks)) = w0;
      if (k0 + 64 < a.k_lo) *reinterpret_cast<uint32_t*>(a.lo_sf + sf_tiled_offset(row, kb + 4, a.lo_chunks)) = w1;
    } else {
      uint8_t* p = a.lo_sf + static_cast<size_t>(row) * (a.k_lo >> 4) + kb;
      if (k0 < a.k_lo) *reinterpret_cast<uint32_t*>(p) = w0;
      if (k0 + 64 < a.k_lo) *reinterpret_cast<uint32_t*>(p + 4) = w1;
    }
  }
  if constexpr (PRO == 3) {
    // the last block to finish closes the call: the counter the next call's handshake is derived from
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(a.sync + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        a.sync[1] = 0;
        __threadfence();
        atomicAdd(a.sync, 1);
      }
    }
  }
}

// ---- dequantise packed -> bf16 [rows, k]; one thread per 8 elements -------------------------
struct UnpackArgs {
  const uint8_t *lo_codes, *lo_sf, *hi_codes, *hi_sf;
  int sf_tiled, rows, k_lo, k_hi, lo_chunks, hi_chunks;
  uint4* y;
};

__global__ void unpack_kernel(const UnpackArgs a) {
  const int k = a.k_lo + a.k_hi;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t per_row = k >> 3;
  if (idx >= per_row * a.rows) return;
  const int row = static_cast<int>(idx / per_row);
  const int kk = static_cast<int>(idx % per_row) * 8;
  float f[8];
  if (kk < a.k_lo) {
    const uint32_t codes = *reinterpret_cast<const uint32_t*>(a.lo_codes + (static_cast<size_t>(row) * a.k_lo + kk) / 2);
    const int kb = kk >> 4;
    const uint8_t sc = a.sf_tiled ? a.lo_sf[sf_tiled_offset(row, kb, a.lo_chunks)]
                                  : a.lo_sf[static_cast<size_t>(row) * (a.k_lo >> 4) + kb];
    const float s = e4m3_code_to_f32(sc);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t c = (codes >> (4 * i)) & 0xF;
      const uint32_t mag = c & 7;
      // E2M1 magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
      const float mv = mag < 2 ? 0.5f * mag : __uint_as_float(((mag >> 1) + 126u) << 23 | (mag & 1u) << 22);
      f[i] = (c & 8) ? -(mv * s) : mv * s;
    }
  } else {
    const int kh = kk - a.k_lo;
    const uint2 codes = *reinterpret_cast<const uint2*>(a.hi_codes + static_cast<size_t>(row) * a.k_hi + kh);
    const int kb = kh >> 5;
    const uint8_t sc = a.sf_tiled ? a.hi_sf[sf_tiled_offset(row, kb, a.hi_chunks)]
                                  : a.hi_sf[static_cast<size_t>(row) * (a.k_hi >> 5) + kb];
    const float s = e8m0_to_f32(sc);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t c = ((i < 4 ? codes.x : codes.y) >> (8 * (i & 3))) & 0xFF;
      const float mv = e4m3_code_to_f32(c & 0x7F);
      f[i] = (c & 0x80) ? -(mv * s) : mv * s;
    }
  }
  uint4 o;
  o.x = f32x2_to_bf16x2(f[0], f[1]); o.y = f32x2_to_bf16x2(f[2], f[3]);
  o.z = f32x2_to_bf16x2(f[4], f[5]); o.w = f32x2_to_bf16x2(f[6], f[7]);
  a.y[idx] = o;
}

static int check_pack_args(const void* x, int64_t rows, int64_t k, int64_t k_hi, int hadamard, bool norm,
                           void* lo_codes, void* lo_sf, void* hi_codes, void* hi_sf, int sf_layout) {
  if (rows < 0 || k <= 0 || k_hi < 0 || k_hi > k) return PLQ_ERR_SHAPE;
  const int64_t k_lo = k - k_hi;
  if (k_lo % 64 != 0 || k_hi % 32 != 0) return PLQ_ERR_SHAPE;
  if ((hadamard || norm) && k % 128 != 0) return PLQ_ERR_SHAPE;
  if (k > 32768) return PLQ_ERR_LIMIT;
  if (rows > 0x7FFFFFFF) return PLQ_ERR_LIMIT;
  if (sf_layout != PLQ_SF_ROWMAJOR && sf_layout != PLQ_SF_TILED) return PLQ_ERR_SHAPE;
  if (rows == 0) return PLQ_OK;   // nothing to read or write: pointers may be anything
  if (!x) return PLQ_ERR_NULL;
  if (k_lo && (!lo_codes || !lo_sf)) return PLQ_ERR_NULL;
  if (k_hi && (!hi_codes || !hi_sf)) return PLQ_ERR_NULL;
  if (!aligned16(x) || !aligned16(lo_codes) || !aligned16(lo_sf) || !aligned16(hi_codes) || !aligned16(hi_sf))
    return PLQ_ERR_ALIGN;
  return PLQ_OK;
}

struct PeerArgs {
  const void* const* peer_x;
  void* const* peer_flags;
  int32_t* flags;
  int32_t* sync;
  int32_t* status;
  int world, rank;
};

static int launch_pack(int pro, const void* x, const void* x2, void* h_out, int64_t ldx, const void* gamma, float eps,
                       int64_t rows, int64_t k, int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf,
                       void* hi_codes, void* hi_sf, int sf_layout, void* stream, const PeerArgs* peers = nullptr) {
  const bool norm = gamma != nullptr;
  if (ldx < k || ldx % 8 != 0) return PLQ_ERR_SHAPE;
  if (rows > 0 && pro != 0 && (!x2 || !aligned16(x2))) return x2 ? PLQ_ERR_ALIGN : PLQ_ERR_NULL;
  if (rows > 0 && pro >= 2 && (!h_out || !aligned16(h_out))) return h_out ? PLQ_ERR_ALIGN : PLQ_ERR_NULL;
  if (pro == 3 && (!peers || !peers->peer_x || !peers->peer_flags || !peers->flags || !peers->sync || !peers->status))
    return PLQ_ERR_NULL;
  if (pro == 3 && (peers->world < 1 || peers->world > 8 || peers->rank < 0 || peers->rank >= peers->world)) return PLQ_ERR_SHAPE;
  int st = check_pack_args(pro == 3 ? x2 : x, rows, k, k_hi, hadamard, norm, lo_codes, lo_sf, hi_codes, hi_sf, sf_layout);
  if (st != PLQ_OK) return st;
  if (rows == 0) return PLQ_OK;
  if (norm && !aligned16(gamma)) return PLQ_ERR_ALIGN;
  st = device_check();
  if (st != PLQ_OK) return st;
  PackArgs a;
  a.x = static_cast<const uint4*>(x);
  a.x2 = static_cast<const uint4*>(x2);
  a.h_out = static_cast<uint4*>(h_out);
  a.ldx8 = static_cast<int>(ldx / 8);
  a.peer_x = nullptr; a.peer_flags = nullptr; a.flags = nullptr; a.sync = nullptr; a.status = nullptr;
  a.world = 1; a.rank = 0;
  if (peers) {
    a.peer_x = reinterpret_cast<const uint4* const*>(peers->peer_x);
    a.peer_flags = reinterpret_cast<int* const*>(peers->peer_flags);
    a.flags = peers->flags; a.sync = peers->sync; a.status = peers->status;
    a.world = peers->world; a.rank = peers->rank;
  }
  a.gamma = static_cast<const uint4*>(gamma);
  a.eps = eps;
  a.rows = static_cast<int>(rows);
  a.k = static_cast<int>(k);
  a.k_lo = static_cast<int>(k - k_hi);
  a.lo_codes = static_cast<uint8_t*>(lo_codes);
  a.lo_sf = static_cast<uint8_t*>(lo_sf);
  a.hi_codes = static_cast<uint8_t*>(hi_codes);
  a.hi_sf = static_cast<uint8_t*>(hi_sf);
  a.sf_tiled = sf_layout == PLQ_SF_TILED;
  a.lo_chunks = static_cast<int>(((k - k_hi) / 16 + 3) / 4);
  a.hi_chunks = static_cast<int>((k_hi / 32 + 3) / 4);
  const int blocks128 = static_cast<int>((k + 127) / 128);
  const int threads = ((blocks128 * 4 + 31) / 32) * 32;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(rows), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  auto launch = [&](void (*kernel)(const PackArgs)) { return cudaLaunchKernelEx(&cfg, kernel, a); };
  if (pro == 1) {                      // SiLU(gate) * up: no norm in front of the down projection
    if (norm) return PLQ_ERR_SHAPE;
    if (hadamard) PLQ_CUDA_TRY(launch(pack_kernel<1, false, true>));
    else PLQ_CUDA_TRY(launch(pack_kernel<1, false, false>));
  } else if (pro == 3) {               // all-reduce over peer memory, residual add, then RMSNorm
    if (!norm) return PLQ_ERR_NULL;
    if (hadamard) PLQ_CUDA_TRY(launch(pack_kernel<3, true, true>));
    else PLQ_CUDA_TRY(launch(pack_kernel<3, true, false>));
  } else if (pro == 2) {               // residual add, then RMSNorm
    if (!norm) return PLQ_ERR_NULL;
    if (hadamard) PLQ_CUDA_TRY(launch(pack_kernel<2, true, true>));
    else PLQ_CUDA_TRY(launch(pack_kernel<2, true, false>));
  } else if (norm && hadamard) PLQ_CUDA_TRY(launch(pack_kernel<0, true, true>));
  else if (norm) PLQ_CUDA_TRY(launch(pack_kernel<0, true, false>));
  else if (hadamard) PLQ_CUDA_TRY(launch(pack_kernel<0, false, true>));
  else PLQ_CUDA_TRY(launch(pack_kernel<0, false, false>));
  return PLQ_OK;
}

}  // namespace plq

extern "C" int plq_pack(const void* x_bf16, int64_t rows, int64_t k, int64_t k_hi, int hadamard, void* lo_codes,
                        void* lo_sf, void* hi_codes, void* hi_sf, int sf_layout, void* stream) {
  return plq::launch_pack(0, x_bf16, nullptr, nullptr, k, nullptr, 0.0f, rows, k, k_hi, hadamard, lo_codes, lo_sf,
                          hi_codes, hi_sf, sf_layout, stream);
}

extern "C" int plq_rmsnorm_pack(const void* x_bf16, const void* gamma_bf16, float eps, int64_t rows, int64_t k,
                                int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf, void* hi_codes,
                                void* hi_sf, int sf_layout, void* stream) {
  if (!gamma_bf16) return PLQ_ERR_NULL;
  return plq::launch_pack(0, x_bf16, nullptr, nullptr, k, gamma_bf16, eps, rows, k, k_hi, hadamard, lo_codes, lo_sf,
                          hi_codes, hi_sf, sf_layout, stream);
}

extern "C" int plq_silu_mul_pack(const void* gate_bf16, const void* up_bf16, int64_t ld, int64_t rows, int64_t k,
                                 int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf, void* hi_codes,
                                 void* hi_sf, int sf_layout, void* stream) {
  return plq::launch_pack(1, gate_bf16, up_bf16, nullptr, ld, nullptr, 0.0f, rows, k, k_hi, hadamard, lo_codes,
                          lo_sf, hi_codes, hi_sf, sf_layout, stream);
}

extern "C" int plq_add_rmsnorm_pack(const void* x_bf16, const void* residual_bf16, void* h_out_bf16,
                                    const void* gamma_bf16, float eps, int64_t rows, int64_t k, int64_t k_hi,
                                    int hadamard, void* lo_codes, void* lo_sf, void* hi_codes, void* hi_sf,
                                    int sf_layout, void* stream) {
  if (!gamma_bf16) return PLQ_ERR_NULL;
  return plq::launch_pack(2, x_bf16, residual_bf16, h_out_bf16, k, gamma_bf16, eps, rows, k, k_hi, hadamard,
                          lo_codes, lo_sf, hi_codes, hi_sf, sf_layout, stream);
}

extern "C" int plq_allreduce_add_rmsnorm_pack(const void* const* peer_x_dev, void* const* peer_flags_dev, int32_t* flags,
                                              int32_t* sync, int world, int rank, const void* residual_bf16,
                                              void* h_out_bf16, const void* gamma_bf16, float eps, int64_t rows,
                                              int64_t k, int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf,
                                              void* hi_codes, void* hi_sf, int sf_layout, int32_t* dev_status,
                                              void* stream) {
  if (!gamma_bf16) return PLQ_ERR_NULL;
  if (rows < 1) return PLQ_ERR_SHAPE;               // every rank must launch, or the others wait for it
  const plq::PeerArgs peers = {peer_x_dev, peer_flags_dev, flags, sync, dev_status, world, rank};
  return plq::launch_pack(3, nullptr, residual_bf16, h_out_bf16, k, gamma_bf16, eps, rows, k, k_hi, hadamard, lo_codes,
                          lo_sf, hi_codes, hi_sf, sf_layout, stream, &peers);
}

extern "C" int plq_unpack(const void* lo_codes, const void* lo_sf, const void* hi_codes, const void* hi_sf,
                          int sf_layout, int64_t rows, int64_t k_lo, int64_t k_hi, void* y_bf16, void* stream) {
  using namespace plq;
  if (rows < 0 || k_lo < 0 || k_hi < 0 || k_lo + k_hi <= 0) return PLQ_ERR_SHAPE;
  if (k_lo % 64 != 0 || k_hi % 32 != 0) return PLQ_ERR_SHAPE;
  if (rows > 0x7FFFFFFF || k_lo + k_hi > (1 << 20)) return PLQ_ERR_LIMIT;
  if (!y_bf16 || (k_lo && (!lo_codes || !lo_sf)) || (k_hi && (!hi_codes || !hi_sf))) return PLQ_ERR_NULL;
  if (!aligned16(y_bf16) || !aligned16(lo_codes) || !aligned16(hi_codes)) return PLQ_ERR_ALIGN;
  int st = device_check();
  if (st != PLQ_OK) return st;
  if (rows == 0) return PLQ_OK;
  UnpackArgs a;
  a.lo_codes = static_cast<const uint8_t*>(lo_codes);
  a.lo_sf = static_cast<const uint8_t*>(lo_sf);
  a.hi_codes = static_cast<const uint8_t*>(hi_codes);
  a.hi_sf = static_cast<const uint8_t*>(hi_sf);
  a.sf_tiled = sf_layout == PLQ_SF_TILED;
  a.rows = static_cast<int>(rows);
  a.k_lo = static_cast<int>(k_lo);
  a.k_hi = static_cast<int>(k_hi);
  a.lo_chunks = static_cast<int>((k_lo / 16 + 3) / 4);
  a.hi_chunks = static_cast<int>((k_hi / 32 + 3) / 4);
  a.y = static_cast<uint4*>(y_bf16);
  const int64_t total = rows * ((k_lo + k_hi) / 8);
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((total + threads - 1) / threads);
  unpack_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PLQ_CUDA_TRY(cudaGetLastError());
  return PLQ_OK;
}
