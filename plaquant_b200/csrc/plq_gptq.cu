// GPTQ inner loop for the block-scaled FP formats: Hessian-corrected rounding of one block of weight columns
// against block scales frozen beforehand (promix/quantize/gptq.py:142-205 with
// quantize_column_with_frozen_scale, promix/quantize/quant_utils.py:616-657, in the reference).
//
// The loop is sequential in the columns and independent in the rows, so a warp owns a row: lane j holds columns
// j, j + 32, j + 64, j + 96 of the block in registers, column i is broadcast from its owner, every lane computes
// its rounding and error, and each lane folds the error into its own later columns.  The block of the inverse
// Hessian factor sits in shared memory.  Arithmetic follows the reference operation by operation in float32:
// IEEE division by the scale, clamp, round to nearest (ties to even) on the element grid, multiply by the scale;
// err = (w - q) / d; w[c] -= err * Hinv[i, c] with the product rounded before the subtraction (the reference's
// rank-one update is a matmul followed by an in-place subtraction).
#include "plq_quant.cuh"

namespace plq {

constexpr int kGptqMaxBlock = 128;
constexpr int kGptqWarps = 4;

struct GptqArgs {
  const float* w;       // [rows, k] row stride ldw: the weights with every earlier block's correction applied
  const float* hinv;    // [k, k] row stride ldh: upper Cholesky factor of the inverse Hessian
  const uint8_t* lo_sf; // [rows, k_lo / 16] E4M3 scale bytes, frozen
  const uint8_t* hi_sf; // [rows, k_hi / 32] E8M0 scale bytes, frozen
  float* q;             // [rows, k] row stride ldq: receives the dequantised columns of the block
  float* err;           // [rows, count]: receives (w - q) / d per column of the block
  uint8_t* codes;       // [rows, k]: receives one code per element (E2M1 in the low nibble, or E4M3)
  int64_t ldw, ldh, ldq;
  int rows, k, k_lo, i1, count;
};

__device__ __forceinline__ float e2m1_code_to_f32(uint32_t c) {
  const uint32_t mag = c & 7u;
  const float mv = mag < 2 ? 0.5f * static_cast<float>(mag) : __uint_as_float(((mag >> 1) + 126u) << 23 | (mag & 1u) << 22);
  return (c & 8u) ? -mv : mv;
}

__global__ void __launch_bounds__(kGptqWarps * 32) gptq_block_kernel(const GptqArgs a) {
  extern __shared__ float hs[];                       // [count][count] block of hinv
  for (int idx = threadIdx.x; idx < a.count * a.count; idx += blockDim.x) {
    const int r = idx / a.count, c = idx - r * a.count;
    hs[idx] = a.hinv[static_cast<size_t>(a.i1 + r) * a.ldh + a.i1 + c];
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kGptqWarps + (threadIdx.x >> 5);
  if (row >= a.rows) return;
  const int k_hi = a.k - a.k_lo;
  float wv[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int c = 32 * t + lane;
    wv[t] = c < a.count ? a.w[static_cast<size_t>(row) * a.ldw + a.i1 + c] : 0.0f;
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    for (int j = 0; j < 32; ++j) {
      const int i = 32 * t + j;
      if (i >= a.count) break;                        // uniform over the warp
      const float w = __shfl_sync(0xFFFFFFFFu, wv[t], j);
      const int col = a.i1 + i;
      float s, qv;
      uint32_t code;
      if (col < a.k_lo) {
        s = e4m3_code_to_f32(a.lo_sf[static_cast<size_t>(row) * (a.k_lo >> 4) + (col >> 4)]);
        const float x = fminf(fmaxf(__fdiv_rn(w, s), -6.0f), 6.0f);
        uint16_t b;
        asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}" : "=h"(b) : "f"(0.0f), "f"(x));
        code = b & 0xFu;
        qv = __fmul_rn(e2m1_code_to_f32(code), s);
      } else {
        s = e8m0_to_f32(a.hi_sf[static_cast<size_t>(row) * (k_hi >> 5) + ((col - a.k_lo) >> 5)]);
        const float x = fminf(fmaxf(__fdiv_rn(w, s), -448.0f), 448.0f);
        code = f32_to_e4m3_rn_sat(x);
        const float mv = e4m3_code_to_f32(code & 0x7Fu);
        qv = __fmul_rn((code & 0x80u) ? -mv : mv, s);
      }
      const float* hrow = hs + i * a.count;
      const float e = __fdiv_rn(__fsub_rn(w, qv), hrow[i]);
      if (lane == j) {
        a.q[static_cast<size_t>(row) * a.ldq + col] = qv;
        a.err[static_cast<size_t>(row) * a.count + i] = e;
        a.codes[static_cast<size_t>(row) * a.k + col] = static_cast<uint8_t>(code);
      }
#pragma unroll
      for (int t2 = 0; t2 < 4; ++t2) {
        const int c = 32 * t2 + lane;
        if (c >= i && c < a.count) wv[t2] = __fsub_rn(wv[t2], __fmul_rn(e, hrow[c]));
      }
    }
  }
}

}  // namespace plq

extern "C" int plq_gptq_block_frozen(const void* w_f32, int64_t ldw, const void* hinv_f32, int64_t ldh,
                                     const void* lo_sf, const void* hi_sf, int64_t rows, int64_t k, int64_t k_hi,
                                     int64_t col0, int64_t count, void* q_f32, int64_t ldq, void* err_f32,
                                     void* codes_u8, void* stream) {
  using namespace plq;
  if (rows < 1 || k < 1 || k_hi < 0 || k_hi > k || col0 < 0 || count < 1 || col0 + count > k) return PLQ_ERR_SHAPE;
  if ((k - k_hi) % 16 != 0 || k_hi % 32 != 0 || ldw < k || ldh < k || ldq < k) return PLQ_ERR_SHAPE;
  if (count > kGptqMaxBlock || rows > 0x7FFFFFFF || k > (1 << 24)) return PLQ_ERR_LIMIT;
  if (!w_f32 || !hinv_f32 || !q_f32 || !err_f32 || !codes_u8) return PLQ_ERR_NULL;
  if ((k - k_hi) && !lo_sf) return PLQ_ERR_NULL;
  if (k_hi && !hi_sf) return PLQ_ERR_NULL;
  int st = device_check();
  if (st != PLQ_OK) return st;
  GptqArgs a;
  a.w = static_cast<const float*>(w_f32); a.hinv = static_cast<const float*>(hinv_f32);
  a.lo_sf = static_cast<const uint8_t*>(lo_sf); a.hi_sf = static_cast<const uint8_t*>(hi_sf);
  a.q = static_cast<float*>(q_f32); a.err = static_cast<float*>(err_f32); a.codes = static_cast<uint8_t*>(codes_u8);
  a.ldw = ldw; a.ldh = ldh; a.ldq = ldq;
  a.rows = static_cast<int>(rows); a.k = static_cast<int>(k); a.k_lo = static_cast<int>(k - k_hi);
  a.i1 = static_cast<int>(col0); a.count = static_cast<int>(count);
  const size_t smem = static_cast<size_t>(count) * count * sizeof(float);
  static thread_local int attr_dev = -1;
  int dev = 0;
  PLQ_CUDA_TRY(cudaGetDevice(&dev));
  if (attr_dev != dev) {
    PLQ_CUDA_TRY(cudaFuncSetAttribute(gptq_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      kGptqMaxBlock * kGptqMaxBlock * 4));
    attr_dev = dev;
  }
  const unsigned grid = static_cast<unsigned>((rows + kGptqWarps - 1) / kGptqWarps);
  gptq_block_kernel<<<grid, kGptqWarps * 32, smem, static_cast<cudaStream_t>(stream)>>>(a);
  PLQ_CUDA_TRY(cudaGetLastError());
  return PLQ_OK;
}
