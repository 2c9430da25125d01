// Quantise-and-pack kernels: [RMSNorm] -> [block-Hadamard 128] -> NVFP4 | MXFP8 codes + scales,
// and the inverse (dequantise to bf16).  HBM-bound elementwise work.
//
// Thread mapping.  A row is cut into 128-element blocks (the Hadamard block) and two consecutive
// lanes own one block: lane l of a row loads the 64 contiguous elements [64 l, 64 l + 64) as two
// runs of 32 (eight 16-byte loads), held as 2 x 16 float32 pairs.  A CTA works on `rows_per_cta`
// rows at once.  In this mapping
//   * butterfly strides 1..16 stay inside a run and stride 32 combines the two runs of a lane, so
//     six of the seven stages need no other lane;
//   * stride 64 pairs the two lanes of a block.  Each lane keeps one run and sends the other: the
//     even lane ends up with the sums and differences of elements [0, 32) u [64, 96) of the block,
//     the odd lane with [32, 64) u [96, 128): 32 shuffles per 64 elements instead of 64.  So that
//     both lanes keep register run 0 and send run 1, the odd lane holds its runs swapped from the
//     load on (run 0 = elements [96, 128)), which the stride-32 stage absorbs in the sign of one
//     multiplier; the odd lane's differences come out negated and the sign returns in the final
//     multiplication by +-1/sqrt(128) (negation is exact, so every element sees the same roundings
//     as in the plain butterfly network);
//   * after the rotation every lane holds two whole runs of 32 consecutive elements: the NVFP4
//     blocks (16) and MXFP8 blocks (32) are lane-local - no shuffle for the block maxima, one
//     scale computation per block, 16-byte code stores;
//   * the NVFP4/MXFP8 boundary (a multiple of 64) never cuts a run.
// Summation and butterfly order are fixed and documented in the CPU oracle
// (`_sumsq_det`, `block_hadamard_det`), which these kernels match bit for bit.
#include <map>
#include <mutex>
#include <tuple>
#include <utility>

#include "plq_quant.cuh"

namespace plq {

#ifndef PLQ_PACK_TARGET_THREADS
#define PLQ_PACK_TARGET_THREADS 128
#endif
constexpr int kPackTargetThreads = PLQ_PACK_TARGET_THREADS;   // CTA size the launcher aims for (whole rows)

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
  int buffer_index;              // which of the two buffer sets peer_x names (0 / 1), or -1: checked against the call count
  // prologue 3, scattered form: this rank handles rows [row0, row0 + rows) of the ranks' [total, k] buffers and
  // stores their packed codes and scales into every rank's output buffers (out_tbl[8 * i + r], i = lo_codes,
  // lo_sf, hi_codes, hi_sf); nullptr = the plain form (all rows, own outputs)
  uint8_t* const* out_tbl;
  int row0;
  const uint4* gamma;    // bf16 [k] (RMSNorm weight) or nullptr
  float eps;
  int rows, k, k_lo;     // k_hi = k - k_lo
  uint8_t* lo_codes;     // [rows, k_lo/2]
  uint8_t* lo_sf;
  uint8_t* hi_codes;     // [rows, k_hi]
  uint8_t* hi_sf;
  int sf_tiled;
  int lo_chunks, hi_chunks;  // chunks per 128-row group in the tiled layouts
  int lanes;                 // threads per row: ceil(k / 64) rounded up to a whole warp
  int rows_per_cta;          // with a row norm: rows per CTA (warps per CTA = rows_per_cta * lanes / 32)
  int ngroups;               // groups of (warps per CTA) work units = ceil(rows * (lanes / 32) / warps per CTA)
  int stages;                // groups of rows in flight per CTA (1..3 shared-memory stages)
};

// Four 32-bit words of bf16 pairs -> four float32 pairs.
__device__ __forceinline__ void unpack8(const uint4& w, float2* v) {
  v[0] = make_float2(bf16lo_to_f32(w.x), bf16hi_to_f32(w.x));
  v[1] = make_float2(bf16lo_to_f32(w.y), bf16hi_to_f32(w.y));
  v[2] = make_float2(bf16lo_to_f32(w.z), bf16hi_to_f32(w.z));
  v[3] = make_float2(bf16lo_to_f32(w.w), bf16hi_to_f32(w.w));
}

// Round a float32 pair to bf16 and widen it again.
__device__ __forceinline__ float2 round_bf16_pair(const float2 y) {
  const uint32_t b = f32x2_to_bf16x2(y.x, y.y);
  return make_float2(bf16lo_to_f32(b), bf16hi_to_f32(b));
}

// Output stores.  Plain: this rank's buffer.  Scattered tensor-parallel prologue (PRO 3 with an output table): the
// same bytes into the buffer of every rank (an all-gather by peer stores over NVLink).  `which` = 0 lo_codes, 1 lo_sf,
// 2 hi_codes, 3 hi_sf.  Only prologue 3 carries the table: the other kernels compile to the plain store.
template <int PRO, typename T>
__device__ __forceinline__ void store_out(const PackArgs& a, int which, uint8_t* own, size_t off, const T& val) {
  if constexpr (PRO == 3) {
    if (a.out_tbl != nullptr) {
      for (int r = 0; r < a.world; ++r) *reinterpret_cast<T*>(a.out_tbl[8 * which + r] + off) = val;
      return;
    }
  }
  *reinterpret_cast<T*>(own + off) = val;
}

// Quantises one NVFP4 run of 32 elements (sixteen float32 pairs, bf16-valued): its 16 bytes of codes go to `codes`,
// its two scale bytes (block order) are returned.
__device__ __forceinline__ uint32_t quantize_run_nvfp4(const float2* v, uint4& codes) {
  uint32_t sf2 = 0;
  uint32_t words[4];
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    float m0 = 0.0f, m1 = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      m0 = fmaxf(m0, fmaxf(fabsf(v[8 * b + i].x), fabsf(v[8 * b + i].y)));
      m1 = fmaxf(m1, fmaxf(fabsf(v[8 * b + i + 1].x), fabsf(v[8 * b + i + 1].y)));
    }
    const uint32_t c = nvfp4_scale_code(fmaxf(m0, m1));
    const float s = e4m3_code_to_f32(c);
    const float r = __frcp_rn(s);
    words[2 * b] = nvfp4_quantize8(v + 8 * b, s, r);
    words[2 * b + 1] = nvfp4_quantize8(v + 8 * b + 4, s, r);
    sf2 |= c << (8 * b);
  }
  codes = make_uint4(words[0], words[1], words[2], words[3]);
  return sf2;
}

// Codes of the run that starts at element `o` of output row `row` (o < k_lo).
template <int PRO>
__device__ __forceinline__ void store_run_nvfp4(const PackArgs& a, const uint4& codes, int row, int o) {
  store_out<PRO>(a, 0, a.lo_codes, (static_cast<size_t>(row) * a.k_lo + o) / 2, codes);
}

// The same for a run in the MXFP8 columns (o >= k_lo): 32 code bytes and one scale byte.
template <int PRO>
__device__ __forceinline__ void quantize_run_mxfp8(const PackArgs& a, const float2* v, int row, int o) {
  float m0 = 0.0f, m1 = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i += 2) {
    m0 = fmaxf(m0, fmaxf(fabsf(v[i].x), fabsf(v[i].y)));
    m1 = fmaxf(m1, fmaxf(fabsf(v[i + 1].x), fabsf(v[i + 1].y)));
  }
  const uint32_t c = mxfp8_scale_code(fmaxf(m0, m1));
  const float inv = __uint_as_float((254u - c) << 23);
  const uint2 c0 = mxfp8_quantize8(v, inv), c1 = mxfp8_quantize8(v + 4, inv);
  const uint2 c2 = mxfp8_quantize8(v + 8, inv), c3 = mxfp8_quantize8(v + 12, inv);
  const int k_hi = a.k - a.k_lo, kh = o - a.k_lo;
  const size_t coff = static_cast<size_t>(row) * k_hi + kh;
  store_out<PRO>(a, 2, a.hi_codes, coff, make_uint4(c0.x, c0.y, c1.x, c1.y));
  store_out<PRO>(a, 2, a.hi_codes, coff + 16, make_uint4(c2.x, c2.y, c3.x, c3.y));
  const int kb = kh >> 5;
  const size_t off = a.sf_tiled ? static_cast<size_t>(sf_tiled_offset(row, kb, a.hi_chunks))
                                : static_cast<size_t>(row) * (k_hi >> 5) + kb;
  store_out<PRO>(a, 3, a.hi_sf, off, static_cast<uint8_t>(c));
}

// ---- staging through shared memory -------------------------------------------------------
// A warp works on one segment of a row: the 32 x 128 bytes its lanes own.  The segment travels global ->
// shared memory as 16-byte asynchronous copies whose global addresses are consecutive across the warp
// (coalesced), into a layout where lane `o` owns line o (128 bytes) with its eight 16-byte chunks XOR-swizzled
// by (o & 7); each lane then reads its own line with conflict-free 16-byte loads.  Copies and reads of a
// segment are warp-local, so only warp barriers order them.  Pieces outside the matrix are zero-filled.
constexpr int kSegBytes = 4096;

__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
// waits until at most `pending` (0..2) of the most recently committed groups are still in flight
__device__ __forceinline__ void cp_async_wait_pending(int pending) {
  if (pending <= 0) asm volatile("cp.async.wait_group 0;" ::: "memory");
  else if (pending == 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
  else asm volatile("cp.async.wait_group 2;" ::: "memory");
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}

// Starts the copy of one segment: `src` = first 16-byte piece of the segment in global memory, `npieces` = how
// many of its 256 pieces exist (0 for a row outside the matrix).  Piece 32 j + lane goes to line 4 j + lane / 8,
// chunk (lane & 7) ^ (line & 7): per lane two fixed offsets (even / odd j) plus 512 j.
__device__ __forceinline__ void stage_segment(uint32_t seg_smem, const uint4* src, int npieces, int lane) {
  const uint32_t q = static_cast<uint32_t>(lane) >> 3;
  const uint32_t x = ((static_cast<uint32_t>(lane) & 7u) ^ q) << 4;
  const uint32_t d_even = seg_smem + q * 128 + x, d_odd = seg_smem + q * 128 + (x ^ 64u);
  const uint4* s = src + lane;
  if (npieces == 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) cp_async16(((j & 1) ? d_odd : d_even) + 512 * j, s + 32 * j);
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool valid = 32 * j + lane < npieces;
      cp_async16_zfill(((j & 1) ? d_odd : d_even) + 512 * j, valid ? s + 32 * j : src, valid);
    }
  }
}

// Tensor-parallel prologue: one segment of x = bf16(sum over the ranks of their partial outputs), float32 in rank
// order so that every rank computes the same bits.  Each rank's 4 KB of the segment is read with consecutive
// addresses across the warp (whole 128-byte lines over NVLink), B pieces of all ranks in flight at a time, and the
// sum goes to shared memory in the layout stage_segment produces.  `off0` = index of the lane's first 16-byte piece.
template <int B, int W>
__device__ __forceinline__ void reduce_segment(uint8_t* seg, const uint4* const* peer_x, int world, size_t off0,
                                               int npieces, int lane) {
  const uint32_t q = static_cast<uint32_t>(lane) >> 3;
  const uint32_t x = ((static_cast<uint32_t>(lane) & 7u) ^ q) << 4;
  uint8_t* d_even = seg + q * 128 + x;
  uint8_t* d_odd = seg + q * 128 + (x ^ 64u);
#pragma unroll
  for (int jb = 0; jb < 8; jb += B) {
    uint4 t[B][W];
#pragma unroll
    for (int jj = 0; jj < B; ++jj) {
      const bool valid = 32 * (jb + jj) + lane < npieces;
#pragma unroll
      for (int r = 0; r < W; ++r) {
        t[jj][r] = make_uint4(0, 0, 0, 0);
        if (r < world && valid)
          asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(t[jj][r].x), "=r"(t[jj][r].y), "=r"(t[jj][r].z), "=r"(t[jj][r].w)
                       : "l"(peer_x[r] + off0 + 32 * (jb + jj))
                       : "memory");
      }
    }
#pragma unroll
    for (int jj = 0; jj < B; ++jj) {
      float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int r = 0; r < W; ++r) {
        if (r < world) {
          const uint32_t tt[4] = {t[jj][r].x, t[jj][r].y, t[jj][r].z, t[jj][r].w};
#pragma unroll
          for (int i = 0; i < 4; ++i)
            acc[i] = __fadd2_rn(acc[i], make_float2(bf16lo_to_f32(tt[i]), bf16hi_to_f32(tt[i])));
        }
      }
      const int j = jb + jj;
      *reinterpret_cast<uint4*>(((j & 1) ? d_odd : d_even) + 512 * j) =
          make_uint4(f32x2_to_bf16x2(acc[0].x, acc[0].y), f32x2_to_bf16x2(acc[1].x, acc[1].y),
                     f32x2_to_bf16x2(acc[2].x, acc[2].y), f32x2_to_bf16x2(acc[3].x, acc[3].y));
    }
  }
}

// The lane's own eight pieces, register run 0 first; `xr` = ((lane & 7) ^ (4 if the runs are swapped)) << 4.
__device__ __forceinline__ void read_line(const uint8_t* seg, int lane, uint32_t xr, uint4 (&w)[8]) {
  const uint8_t* line = seg + lane * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) w[c] = *reinterpret_cast<const uint4*>(line + ((16u * c) ^ xr));
}

// PRO selects what is quantised: 0 = x; 1 = SiLU(x) * x2 (gate and up halves of the MLP, rounded to bf16 after
// the activation and after the product like the two PyTorch ops they replace, inference/forward_pass.py:266
// in the reference); 2 = x2 + x (residual add, one rounding, also written to h_out: forward_pass.py:258-262);
// 3 = like 2 with x = bf16(sum over the tensor-parallel ranks of their partial outputs), float32 sum in rank order,
// read from the peers' memory: the all-reduce after a row-parallel linear, the residual add, the norm and the
// quantiser of the next linear in one kernel.
//
// Persistent: a CTA walks over groups of work units (one row segment per warp) with a grid stride.  While a
// group is computed from registers, the next groups' segments are already on their way into shared memory.
// Register budget: without a prologue the kernel gets 96 registers per thread (a bound of 640 threads) so that five
// 128-thread CTAs share an SM (measured 3 % faster than four); the prologues need more and keep 128.
#ifdef PLQ_PACK_MAXNREG
#define PLQ_PACK_BOUNDS __maxnreg__(PLQ_PACK_MAXNREG)
#else
#define PLQ_PACK_BOUNDS __launch_bounds__(PRO == 0 ? 640 : 512)
#endif
template <int PRO, bool NORM, bool HAD>
__global__ void PLQ_PACK_BOUNDS pack_kernel(const PackArgs a) {
  extern __shared__ __align__(1024) uint8_t pack_smem[];
  // Programmatic dependent launch on both sides.  A consumer launched with programmatic stream serialisation
  // (GEMM, decode GEMV) may set itself up and prefetch its weights while this kernel runs; it waits for this
  // grid's completion before reading the codes.  This kernel itself may be launched before its predecessor
  // has finished, and waits here before it reads anything.
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int wpr = a.lanes >> 5;                     // warps (segments) per row
  // Work unit = one segment of one row; unit u = row * wpr + segment.  Group g of a CTA with W warps holds units
  // [g W, g W + W), one per warp.  Kernels with a row norm get W = rows_per_cta * wpr from the launcher, so that the
  // warps of a row share a CTA and warp w always has segment w % wpr of the CTA's row w / wpr; the others may cut
  // rows anywhere (a decode batch of 16 long rows still fills the GPU).
  const int rl = warp / wpr;                        // with a row norm: which of the CTA's rows
  const int p = lane & 1;
  const int flip = HAD ? p : 0;                     // odd lanes of a rotated row hold their runs swapped
  const int k8 = a.k >> 3;
  const uint32_t xr = static_cast<uint32_t>((lane & 7) ^ (4 * flip)) << 4;   // chunk swizzle of this lane's line, run 0 first
  struct Unit { int row, seg; };
  auto unit_of = [&](int group) {
    const int u = group * nwarps + warp;
    Unit t;
    t.row = u / wpr;
    t.seg = u - t.row * wpr;
    return t;
  };
  constexpr bool kStageX = true;                    // x always passes through shared memory ...
  constexpr bool kCopyX = PRO != 3;                 // ... copied there, or (prologue 3) summed there from the peers
  constexpr bool kStageX2 = PRO != 0;
  constexpr int kOperands = (kStageX ? 1 : 0) + (kStageX2 ? 1 : 0);
  const int stage_bytes = kOperands * nwarps * kSegBytes;           // one group of rows, all staged operands
  uint8_t* xs0 = pack_smem + warp * kSegBytes;                       // stage 0; stage s is s * stage_bytes further
  uint8_t* x2s0 = pack_smem + ((kStageX ? nwarps : 0) + warp) * kSegBytes;
  uint8_t* gs = pack_smem + a.stages * stage_bytes + (warp - rl * wpr) * 2 * kSegBytes;   // gamma as float32, this warp's segment
  const int ld2 = PRO == 1 ? a.ldx8 : k8;           // row stride of x2 in 16-byte units

  auto stage_group = [&](int group, int slot) {
    const Unit t = unit_of(group);
    const int n = t.row < a.rows ? min(max(k8 - 256 * t.seg, 0), 256) : 0;     // 16-byte pieces of the segment inside the row
    const size_t r0 = static_cast<size_t>(t.row < a.rows ? t.row : 0);
    if constexpr (kCopyX) stage_segment(smem_u32(xs0 + slot * stage_bytes), a.x + r0 * a.ldx8 + 256 * t.seg, n, lane);
    if constexpr (kStageX2) stage_segment(smem_u32(x2s0 + slot * stage_bytes), a.x2 + r0 * ld2 + 256 * t.seg, n, lane);
  };

  if constexpr (PRO == 3) {
    // Cross-rank handshake.  Call number c = completed calls + 1.  This rank's partial output was written by
    // the preceding kernel of the stream; block 0 announces it by storing c into flags[rank] of every peer, and
    // every block waits (bounded) until all peers have announced c in this rank's flags.  Buffers alternate
    // between two per call site order, so a peer that runs ahead never overwrites what is being read here.
    const int call = *reinterpret_cast<volatile int*>(a.sync) + 1;
    // call c reads buffer set (c + 1) % 2; anything else means the caller broke the alternation (for instance a
    // replayed graph with an odd number of calls) and a peer may still be reading the set that was just rewritten
    if (blockIdx.x == 0 && tid == 0 && a.buffer_index >= 0 && ((call + 1) & 1) != a.buffer_index)
      atomicExch(a.status, PLQ_DEV_PROTOCOL);
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

  const int ngroups = a.ngroups;
  int group = blockIdx.x;
  if constexpr (NORM) {
    // The norm weights, widened to float32 once per CTA: lane `lane` of segment `seg` finds its 64 values, in its
    // own register order, as sixteen 16-byte pieces at gs + (16 c + ...): piece c of all 32 lanes is contiguous.
    if (rl == 0) {
      const int gl = 32 * (warp - rl * wpr) + lane;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int e = 64 * gl + (c < 4 ? 32 * flip : 32 - 32 * flip) + 8 * (c & 3);
        const uint4 gq = e < a.k ? __ldg(a.gamma + (e >> 3)) : make_uint4(0, 0, 0, 0);
        float2 g[4];
        unpack8(gq, g);
        float4* dst = reinterpret_cast<float4*>(gs) + (2 * c) * 32 + lane;
        dst[0] = make_float4(g[0].x, g[0].y, g[1].x, g[1].y);
        dst[32] = make_float4(g[2].x, g[2].y, g[3].x, g[3].y);
      }
    }
  }
  const int stride = static_cast<int>(gridDim.x);
  for (int s = 0; s < a.stages; ++s) {               // fill the ring: one committed copy group per stage
    if (group + s * stride < ngroups) stage_group(group + s * stride, s);
    cp_async_commit();
  }
  int iter = 0, slot = 0;

  for (; group < ngroups; group += stride, ++iter) {
    const Unit unit = unit_of(group);
    const int row = unit.row;
    const int l = 32 * unit.seg + lane;               // lane of the row: elements [64 l, 64 l + 64)
    const int in0 = 64 * l + 32 * flip;               // first element of register run 0 / run 1 as loaded
    const int in1 = 64 * l + 32 - 32 * flip;
    const bool row_ok = row < a.rows;
    const bool ok0 = row_ok && in0 < a.k, ok1 = row_ok && in1 < a.k;
    // v[16 r + 4 c + i] holds elements (8 c + 2 i, 8 c + 2 i + 1) of register run r.  Arithmetic on pairs uses the
    // packed float32x2 instructions of sm_100 (same IEEE rounding per element, half the issue slots).
    float2 v[32];
    int cur_slot;

    // ---- this group's pieces: shared memory -> registers; then the next group's copies start ----------
    {
      uint4 w[8], w2[8];
      cp_async_wait_pending(a.stages - 1);          // the oldest group in flight is this one
      if (NORM && iter == 0) __syncthreads();       // gamma was staged by the warps of the CTA's first row
      else __syncwarp();
      if constexpr (PRO == 3) {
        // this warp's segment of x, summed over the ranks into the x slot (warp-local, like the copies)
        const int n = row_ok ? min(max(k8 - 256 * unit.seg, 0), 256) : 0;
        const size_t off0 = static_cast<size_t>(row_ok ? row + a.row0 : 0) * k8 + 256 * unit.seg + lane;
        const uint4* const* px = a.peer_x;
        if (a.world <= 4) reduce_segment<4, 4>(xs0 + slot * stage_bytes, px, a.world, off0, n, lane);
        else reduce_segment<2, 8>(xs0 + slot * stage_bytes, px, a.world, off0, n, lane);
        __syncwarp();
      }
      if constexpr (kStageX) read_line(xs0 + slot * stage_bytes, lane, xr, w);
      if constexpr (kStageX2) read_line(x2s0 + slot * stage_bytes, lane, xr, w2);
      __syncwarp();                                 // every lane has its pieces: the slot is free again
      if (group + a.stages * stride < ngroups) stage_group(group + a.stages * stride, slot);
      cp_async_commit();
      cur_slot = slot;
      if (++slot == a.stages) slot = 0;
      if constexpr (PRO == 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) unpack8(w[c], v + 4 * c);
      } else if constexpr (PRO == 1) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
          const uint32_t uu[4] = {w2[c].x, w2[c].y, w2[c].z, w2[c].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 sl = silu_det2(make_float2(bf16lo_to_f32(ww[i]), bf16hi_to_f32(ww[i])));
            const uint32_t t = f32x2_to_bf16x2(sl.x, sl.y);                                                        // SiLU, to bf16
            const float2 prod = __fmul2_rn(make_float2(bf16lo_to_f32(t), bf16hi_to_f32(t)),
                                           make_float2(bf16lo_to_f32(uu[i]), bf16hi_to_f32(uu[i])));
            v[4 * c + i] = round_bf16_pair(prod);                                                                  // product, to bf16
          }
        }
      } else {
        uint4* hrow = a.h_out + static_cast<size_t>(row) * k8;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint32_t ww[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
          const uint32_t rr[4] = {w2[c].x, w2[c].y, w2[c].z, w2[c].w};
          uint32_t hh[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 sum = __fadd2_rn(make_float2(bf16lo_to_f32(rr[i]), bf16hi_to_f32(rr[i])),
                                          make_float2(bf16lo_to_f32(ww[i]), bf16hi_to_f32(ww[i])));
            hh[i] = f32x2_to_bf16x2(sum.x, sum.y);
            v[4 * c + i] = make_float2(bf16lo_to_f32(hh[i]), bf16hi_to_f32(hh[i]));
          }
          if (c < 4 ? ok0 : ok1) hrow[((c < 4 ? in0 : in1) >> 3) + (c & 3)] = make_uint4(hh[0], hh[1], hh[2], hh[3]);
        }
      }
    }

    // ---- RMSNorm (inference/forward_pass.py:33-39 in the reference) ------------------------
    if constexpr (NORM) {
      __shared__ float warp_sums[2][16];
      float2 s0 = make_float2(0.0f, 0.0f), s1 = make_float2(0.0f, 0.0f);   // per run: even and odd elements apart
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        s0 = __ffma2_rn(v[i], v[i], s0);                  // v*v is exact for bf16 inputs
        s1 = __ffma2_rn(v[16 + i], v[16 + i], s1);
      }
      float s = __fadd_rn(__fadd_rn(s0.x, s0.y), __fadd_rn(s1.x, s1.y));   // symmetric in the two runs
      s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 1);
      s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 2);
      s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 4);
      s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 8);
      s = s + __shfl_xor_sync(0xFFFFFFFFu, s, 16);             // 32 lanes = 2048 elements, pairwise tree
      float* sums = warp_sums[iter & 1];                       // two sets: one barrier per group is enough
      if (lane == 0) sums[warp] = s;
      asm volatile("bar.sync %0, %1;" ::"r"(rl + 1), "r"(a.lanes) : "memory");   // the warps of this row only
      float tot = 0.0f;
      for (int w = 0; w < wpr; ++w) tot = tot + sums[rl * wpr + w];   // left to right
      const float var = __fdiv_rn(tot, static_cast<float>(a.k));
      const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
      const float2 r2 = make_float2(r, r);
      const float4* gl = reinterpret_cast<const float4*>(gs) + lane;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float4 g = gl[32 * c];
        v[2 * c] = round_bf16_pair(__fmul2_rn(make_float2(g.x, g.y), __fmul2_rn(v[2 * c], r2)));
        v[2 * c + 1] = round_bf16_pair(__fmul2_rn(make_float2(g.z, g.w), __fmul2_rn(v[2 * c + 1], r2)));
      }
    }

    // ---- block-Hadamard(128): strides 1..16 inside a run, 32 across the runs, 64 across the lane pair ----
    if constexpr (HAD) {
      const float2 neg1 = make_float2(-1.0f, -1.0f);
#pragma unroll
      for (int i = 0; i < 32; ++i) {                       // stride 1: inside a pair
        const float x0 = v[i].x, x1 = v[i].y;
        v[i] = make_float2(__fadd_rn(x0, x1), __fsub_rn(x0, x1));
      }
#pragma unroll
      for (int h = 1; h < 16; h <<= 1) {                   // strides 2, 4, 8, 16: pairs i, i + h of one run
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if ((i & h) == 0) {
            const float2 x0 = v[i], x1 = v[i + h];
            v[i] = __fadd2_rn(x0, x1);
            v[i + h] = __ffma2_rn(x1, neg1, x0);           // x0 - x1: exact product, one rounding
          }
        }
      }
      {                                                    // stride 32: run 0 with run 1
        // even lane: run 0 = lower elements: (P, Q) -> (P + Q, P - Q); odd lane: run 0 = upper: (P, Q) -> (Q - P, Q + P)
        const float sg = p ? -1.0f : 1.0f;
        const float2 sp = make_float2(sg, sg), sn = make_float2(-sg, -sg);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 P = v[i], Q = v[16 + i];
          v[i] = __ffma2_rn(P, sp, Q);
          v[16 + i] = __ffma2_rn(Q, sn, P);
        }
      }
      {                                                    // stride 64: keep run 0, trade run 1 with the other lane
        const float c = 0.088388347648318441f;             // 1/sqrt(128), then to bf16
        const float2 c0 = make_float2(c, c), c1 = make_float2(p ? -c : c, p ? -c : c);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 o;
          o.x = __shfl_xor_sync(0xFFFFFFFFu, v[16 + i].x, 1);
          o.y = __shfl_xor_sync(0xFFFFFFFFu, v[16 + i].y, 1);
          const float2 k = v[i];
          const float2 sum = __fadd2_rn(k, o);             // elements [32 p, 32 p + 32) of the block
          const float2 dif = __ffma2_rn(o, neg1, k);       // elements [64 + 32 p, ...): negated in the odd lane
          v[i] = round_bf16_pair(__fmul2_rn(sum, c0));
          v[16 + i] = round_bf16_pair(__fmul2_rn(dif, c1));
        }
      }
    }

    // ---- quantise: two runs of 32 consecutive elements per lane -------------------------------
    // first element of the run now in v[0..15] / v[16..31]
    const int o0 = HAD ? 128 * (l >> 1) + 32 * p : 64 * l;
    const int o1 = HAD ? o0 + 64 : o0 + 32;
    uint32_t sf;
    const int orow = PRO == 3 ? row + a.row0 : row;  // row of the outputs (the scattered prologue works on a slice)
    const bool hi0 = o0 >= a.k_lo && o0 < a.k, hi1 = o1 >= a.k_lo && o1 < a.k;
    uint4 c0, c1;
    if (!__any_sync(0xFFFFFFFFu, hi0 || hi1)) {     // the usual case: the whole warp is in the NVFP4 columns
      bool gather = false;                           // scattered form of prologue 3: stores go to every rank
      if constexpr (PRO == 3) gather = a.out_tbl != nullptr;
      sf = quantize_run_nvfp4(v, c0);
      if (!gather && row_ok && o0 < a.k_lo) store_run_nvfp4<PRO>(a, c0, orow, o0);
      sf |= quantize_run_nvfp4(v + 16, c1) << 16;
      if (!gather && row_ok && o1 < a.k_lo) store_run_nvfp4<PRO>(a, c1, orow, o1);
      if constexpr (PRO == 3) {
        if (gather) {
          // The warp's 1 KB of codes goes to every rank.  Each lane holds two 16-byte pieces that are not
          // neighbours of the next lane's; they pass through the warp's (now free) x slot so that one store
          // instruction covers 512 consecutive bytes - whole lines over NVLink instead of half sectors.
          uint8_t* sc = xs0 + cur_slot * stage_bytes;
          const int seg0 = 2048 * unit.seg;
          const int q0 = (o0 - seg0) >> 5, q1 = (o1 - seg0) >> 5;           // piece index inside the segment
          *reinterpret_cast<uint4*>(sc + 16 * (q0 ^ ((q0 >> 2) & 2))) = c0;
          *reinterpret_cast<uint4*>(sc + 16 * (q1 ^ ((q1 >> 2) & 2))) = c1;
          __syncwarp();
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const int q = 32 * half + lane;
            const uint4 val = *reinterpret_cast<const uint4*>(sc + 16 * (q ^ ((q >> 2) & 2)));
            const int o = seg0 + 32 * q;
            if (row_ok && o < a.k_lo) {
              const size_t off = (static_cast<size_t>(orow) * a.k_lo + o) / 2;
              for (int r = 0; r < a.world; ++r) *reinterpret_cast<uint4*>(a.out_tbl[r] + off) = val;
            }
          }
          __syncwarp();                                // the slot is summed into again only after this
        }
      }
    } else {                                         // a warp that holds MXFP8 columns
      sf = 0;
      if (o0 < a.k_lo) {
        sf = quantize_run_nvfp4(v, c0);
        if (row_ok) store_run_nvfp4<PRO>(a, c0, orow, o0);
      } else if (hi0 && row_ok) quantize_run_mxfp8<PRO>(a, v, orow, o0);
      if (o1 < a.k_lo) {
        sf |= quantize_run_nvfp4(v + 16, c1) << 16;
        if (row_ok) store_run_nvfp4<PRO>(a, c1, orow, o1);
      } else if (hi1 && row_ok) quantize_run_mxfp8<PRO>(a, v + 16, orow, o1);
    }
    // NVFP4 scale bytes, one 32-bit word per 64 elements.  Plain rows: the lane's own four bytes.  Rotated rows:
    // the even lane has bytes 0,1 of both words of its block and the odd lane bytes 2,3: one exchange, one word each.
    if constexpr (HAD) {
      const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, sf, 1);
      sf = p ? __byte_perm(sf, other, 0x3276) : __byte_perm(sf, other, 0x5410);
    }
    if (row_ok && 64 * l < a.k_lo) {
      const int kb = 4 * l;
      const size_t off = a.sf_tiled ? static_cast<size_t>(sf_tiled_offset(orow, kb, a.lo_chunks))
                                    : static_cast<size_t>(orow) * (a.k_lo >> 4) + kb;
      store_out<PRO>(a, 1, a.lo_sf, off, sf);
    }
  }
  cp_async_wait_all();
  if constexpr (PRO == 3) {
    // The last block to finish closes the call: the counter the next call's handshake is derived from.  In the
    // scattered form it first tells every peer that this rank's rows are in place everywhere and waits (bounded)
    // for the same word from all of them: when this grid completes, the rank's buffers hold every rank's rows
    // and no peer reads this rank's partial sums any more.
    if (a.out_tbl != nullptr) __threadfence_system();      // this thread's peer stores before the CTA's hand-in
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      if (atomicAdd(a.sync + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        a.sync[1] = 0;
        if (a.out_tbl != nullptr) {
          const int call = *reinterpret_cast<volatile int*>(a.sync) + 1;
          __threadfence_system();
          for (int r = 0; r < a.world; ++r)
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(a.peer_flags[r] + 32 + a.rank), "r"(call) : "memory");
          const long long t0 = clock64();
          for (int r = 0; r < a.world; ++r) {
            int seen;
            do {
              asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(a.flags + 32 + r) : "memory");
              if (seen - call >= 0) break;
              if (clock64() - t0 > kWaitLimitCycles) {
                atomicExch(a.status, PLQ_DEV_TIMEOUT);
                break;
              }
            } while (true);
          }
        }
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

// CTAs of `kernel` that fit one SM with this block size and dynamic shared memory, looked up once per
// (device, kernel, configuration); the first use on a device also raises the kernel's shared-memory limit.
static int resident_ctas(const void* kernel, int threads, int smem, int* per_sm) {
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, int, int>, int> cache;
  static std::map<std::pair<int, const void*>, bool> raised;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  if (!raised[{dev, kernel}]) {
    cudaFuncAttributes fa;
    PLQ_CUDA_TRY(cudaFuncGetAttributes(&fa, kernel));
    PLQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      227 * 1024 - static_cast<int>(fa.sharedSizeBytes)));
    raised[{dev, kernel}] = true;
  }
  const auto key = std::make_tuple(dev, kernel, threads, smem);
  auto it = cache.find(key);
  if (it == cache.end()) {
    int n = 0;
    PLQ_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, static_cast<size_t>(smem)));
    if (n < 1) return PLQ_ERR_LIMIT;
    it = cache.emplace(key, n).first;
  }
  *per_sm = it->second;
  return PLQ_OK;
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
  int world, rank, buffer_index;
  uint8_t* const* out_tbl;   // scattered form: device array [32] of output addresses, see PackArgs
  int row0;
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
  a.world = 1; a.rank = 0; a.buffer_index = -1; a.out_tbl = nullptr; a.row0 = 0;
  if (peers) {
    a.peer_x = reinterpret_cast<const uint4* const*>(peers->peer_x);
    a.peer_flags = reinterpret_cast<int* const*>(peers->peer_flags);
    a.flags = peers->flags; a.sync = peers->sync; a.status = peers->status;
    a.world = peers->world; a.rank = peers->rank; a.buffer_index = peers->buffer_index;
    a.out_tbl = peers->out_tbl; a.row0 = peers->row0;
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
  // threads per row: one per 64 elements, whole warps.  With a row norm a CTA holds whole rows: as many as fit the
  // target CTA size, fewer when the groups would not cover the GPU a few times over (decode batches).  Without one
  // the unit of work is a row segment (one warp) and a CTA takes any `warps` of them.
  const int lanes = ((static_cast<int>((k + 63) / 64) + 31) / 32) * 32;
  const int wpr = lanes / 32;
  const int64_t units = rows * wpr;
  int warps;
  if (norm) {
    int rpc = kPackTargetThreads / lanes;
    if (rpc < 1) rpc = 1;
    if (rpc > 8) rpc = 8;                               // one named barrier per row of the CTA
    while (rpc > 1 && (rows + rpc - 1) / rpc < 4 * static_cast<int64_t>(sm_count())) rpc >>= 1;
    a.rows_per_cta = rpc;
    warps = rpc * wpr;
  } else {
    warps = kPackTargetThreads / 32;
    while (warps > 1 && (units + warps - 1) / warps < 4 * static_cast<int64_t>(sm_count())) warps >>= 1;
    a.rows_per_cta = 0;
  }
  a.lanes = lanes;
  const int threads = 32 * warps;
  const int64_t groups = (units + warps - 1) / warps;
  a.ngroups = static_cast<int>(groups);
  // shared memory: `stages` groups of rows in flight (each: the staged operands of all warps) + gamma.  Kernels
  // that do little arithmetic per byte (no norm) need more bytes in flight to cover the HBM latency.
  const int stage_bytes = (1 + (pro != 0)) * (threads / 32) * kSegBytes;
  const int gamma_bytes = norm ? (lanes / 32) * 2 * kSegBytes : 0;      // float32 copy of the norm weights
#ifndef PLQ_PACK_MAX_STAGES
#define PLQ_PACK_MAX_STAGES 3
#endif
#ifndef PLQ_PACK_CTAS_PER_SM
#define PLQ_PACK_CTAS_PER_SM 5
#endif
  int stages = (pro == 0 && !norm) ? 3 : 2;
  if (stages > PLQ_PACK_MAX_STAGES) stages = PLQ_PACK_MAX_STAGES;
  const int ctas_per_sm = pro == 0 ? PLQ_PACK_CTAS_PER_SM : 4;       // what the register budgets allow
  while (stages > 1 && ctas_per_sm * (stages * stage_bytes + gamma_bytes + 1024) > 224 * 1024) --stages;
  a.stages = stages;
  const int smem = stages * stage_bytes + gamma_bytes;
  auto launch = [&](void (*kernel)(const PackArgs)) -> int {
    int per_sm = 0;
    const int st = resident_ctas(reinterpret_cast<const void*>(kernel), threads, smem, &per_sm);
    if (st != PLQ_OK) return st;
    const int64_t resident = static_cast<int64_t>(per_sm) * sm_count();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(groups < resident ? groups : resident), 1, 1);   // persistent: grid stride over the groups
    cfg.blockDim = dim3(static_cast<unsigned>(threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PLQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, a));
    return PLQ_OK;
  };
  int st2 = PLQ_OK;
  if (pro == 1) {                      // SiLU(gate) * up: no norm in front of the down projection
    if (norm) return PLQ_ERR_SHAPE;
    st2 = hadamard ? launch(pack_kernel<1, false, true>) : launch(pack_kernel<1, false, false>);
  } else if (pro == 3) {               // all-reduce over peer memory, residual add, then RMSNorm
    if (!norm) return PLQ_ERR_NULL;
    st2 = hadamard ? launch(pack_kernel<3, true, true>) : launch(pack_kernel<3, true, false>);
  } else if (pro == 2) {               // residual add, then RMSNorm
    if (!norm) return PLQ_ERR_NULL;
    st2 = hadamard ? launch(pack_kernel<2, true, true>) : launch(pack_kernel<2, true, false>);
  } else if (norm) {
    st2 = hadamard ? launch(pack_kernel<0, true, true>) : launch(pack_kernel<0, true, false>);
  } else {
    st2 = hadamard ? launch(pack_kernel<0, false, true>) : launch(pack_kernel<0, false, false>);
  }
  return st2;
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
                                              int32_t* sync, int world, int rank, int buffer_index,
                                              const void* residual_bf16,
                                              void* h_out_bf16, const void* gamma_bf16, float eps, int64_t rows,
                                              int64_t k, int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf,
                                              void* hi_codes, void* hi_sf, int sf_layout, int32_t* dev_status,
                                              void* stream) {
  if (!gamma_bf16) return PLQ_ERR_NULL;
  if (rows < 1) return PLQ_ERR_SHAPE;               // every rank must launch, or the others wait for it
  if (buffer_index < -1 || buffer_index > 1) return PLQ_ERR_SHAPE;
  const plq::PeerArgs peers = {peer_x_dev, peer_flags_dev, flags, sync, dev_status, world, rank, buffer_index, nullptr, 0};
  return plq::launch_pack(3, nullptr, residual_bf16, h_out_bf16, k, gamma_bf16, eps, rows, k, k_hi, hadamard, lo_codes,
                          lo_sf, hi_codes, hi_sf, sf_layout, stream, &peers);
}

namespace plq {
// Row-major scale bytes [rows, n_sf] -> the tiled layout the GEMM reads, one 32-bit word (four scales of one row)
// per thread, consecutive threads writing consecutive words of a 512-byte chunk.  Scales beyond n_sf and rows beyond
// `rows` inside the last 128-row group are written as zero.
__global__ void __launch_bounds__(256) tile_sf_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                      int rows, int n_sf, int chunks, long long words) {
  const long long w = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (w >= words) return;
  const int in_chunk = static_cast<int>(w & 127);             // (r & 31) * 4 + ((r >> 5) & 3)
  const long long chunk_id = w >> 7;                           // (r >> 7) * chunks + kb / 4
  const int c = static_cast<int>(chunk_id % chunks);
  const int r = static_cast<int>(chunk_id / chunks) * 128 + (in_chunk & 3) * 32 + (in_chunk >> 2);
  uint32_t v = 0;
  if (r < rows) {
    const uint8_t* p = src + static_cast<size_t>(r) * n_sf + 4 * c;
    if (4 * c + 4 <= n_sf && (n_sf & 3) == 0) v = *reinterpret_cast<const uint32_t*>(p);
    else
      for (int i = 0; i < 4 && 4 * c + i < n_sf; ++i) v |= static_cast<uint32_t>(p[i]) << (8 * i);
  }
  reinterpret_cast<uint32_t*>(dst)[w] = v;
}

static int launch_tile_sf(const void* src, void* dst, int64_t rows, int64_t n_sf, cudaStream_t stream) {
  if (n_sf == 0) return PLQ_OK;
  const int64_t chunks = (n_sf + 3) / 4;
  const long long words = ((rows + 127) / 128) * chunks * 128;
  tile_sf_kernel<<<static_cast<unsigned>((words + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), static_cast<int>(rows), static_cast<int>(n_sf),
      static_cast<int>(chunks), words);
  return cudaGetLastError() == cudaSuccess ? PLQ_OK : PLQ_ERR_CUDA;
}
}  // namespace plq

extern "C" int plq_reduce_scatter_add_rmsnorm_pack(const void* const* peer_x_dev, void* const* peer_flags_dev,
                                                   int32_t* flags, int32_t* sync, int world, int rank, int buffer_index,
                                                   void* const* out_tbl_dev, int64_t row0, int64_t total_rows,
                                                   const void* residual_bf16, void* h_out_bf16, const void* gamma_bf16,
                                                   float eps, int64_t rows, int64_t k, int64_t k_hi, int hadamard,
                                                   void* lo_codes, void* lo_sf_rowmajor, void* hi_codes,
                                                   void* hi_sf_rowmajor, void* lo_sf_tiled, void* hi_sf_tiled,
                                                   int32_t* dev_status, void* stream) {
  if (!gamma_bf16 || !out_tbl_dev) return PLQ_ERR_NULL;
  if (rows < 1 || row0 < 0 || row0 + rows > total_rows || total_rows > 0x7FFFFFFF) return PLQ_ERR_SHAPE;
  if (buffer_index < -1 || buffer_index > 1) return PLQ_ERR_SHAPE;
  if ((lo_sf_tiled != nullptr) != (hi_sf_tiled != nullptr || k_hi == 0)) return PLQ_ERR_NULL;
  if (lo_sf_tiled && ((reinterpret_cast<uintptr_t>(lo_sf_tiled) | reinterpret_cast<uintptr_t>(hi_sf_tiled)) & 15))
    return PLQ_ERR_ALIGN;
  const plq::PeerArgs peers = {peer_x_dev, peer_flags_dev, flags, sync, dev_status, world, rank, buffer_index,
                               reinterpret_cast<uint8_t* const*>(out_tbl_dev), static_cast<int>(row0)};
  // the kernel gathers the scale bytes row-major (whole lines per warp over NVLink); the GEMM's tiled copy is
  // made locally afterwards, for all rows, once the kernel has seen every rank finish
  int st = plq::launch_pack(3, nullptr, residual_bf16, h_out_bf16, k, gamma_bf16, eps, rows, k, k_hi, hadamard, lo_codes,
                            lo_sf_rowmajor, hi_codes, hi_sf_rowmajor, PLQ_SF_ROWMAJOR, stream, &peers);
  if (st != PLQ_OK || !lo_sf_tiled) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  st = plq::launch_tile_sf(lo_sf_rowmajor, lo_sf_tiled, total_rows, (k - k_hi) / 16, cs);
  if (st == PLQ_OK) st = plq::launch_tile_sf(hi_sf_rowmajor, hi_sf_tiled, total_rows, k_hi / 32, cs);
  return st;
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
