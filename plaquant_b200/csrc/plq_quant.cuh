// Device arithmetic of the NVFP4 / MXFP8 quantiser.
//
// Every function reproduces, bit for bit on bf16-valued inputs, what the reference's float32
// fake quantiser computes (promix/quantize/quant_utils.py:660-751), but without its
// 127-entry table scans and IEEE divisions:
//   * NVFP4 scale:  smallest E4M3 value s with s >= fl(max/6).  For a bf16 max this is the
//     smallest s with 6*s >= max (6*s is exact in float32 and a bf16 value can never sit
//     within float32 rounding distance of 6*s without being equal to it), so a hardware
//     round-to-nearest conversion plus one exact comparison finds it.
//   * NVFP4 element: E2M1 code of fl(x/s).  x*fl(1/s) refined by one Newton step
//     (two FMAs) equals m exactly whenever x == m*s for a rounding midpoint m, and is far
//     (>= 2^-9 relative) from every midpoint otherwise, so the hardware RNE conversion of
//     the refined quotient yields the same code as the reference's correctly rounded one.
//   * MXFP8 scale: 2^e with the smallest e such that 448*2^e >= max, read off the bf16
//     exponent and mantissa; element: x * 2^-e is exact, then hardware RNE to E4M3.
//   * sign of zero: the reference multiplies the rounded magnitude by sign(x/s), so only a
//     quotient that is strictly negative gets the sign bit.
// The GPU parity tests sweep every (scale, bf16 value) pair against the CPU oracle.
#pragma once

#include "plq_common.cuh"

namespace plq {
#ifdef __CUDACC__

// two bf16 in one 32-bit word -> float32 (element 0 in the low half)
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// round two float32 to bf16 (nearest even) and return them packed (a in the low half)
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float a, float b) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(b), "f"(a));
  return d;
}

// E4M3 code (0..0x7E) -> float32, subnormals included: the code shifted into the float32
// exponent/mantissa position is the value scaled by 2^-120 (a float32 subnormal for codes < 8).
__device__ __forceinline__ float e4m3_code_to_f32(uint32_t c) {
  return __uint_as_float(c << 20) * 1.329227995784916e36f;  // 2^120
}

__device__ __forceinline__ uint32_t f32_to_e4m3_rn_sat(float v) {
  uint16_t d;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(0.0f), "f"(v));
  return d & 0xFFu;
}

// NVFP4 block scale code from the block's absolute maximum (bf16-valued, >= 0, finite).
__device__ __forceinline__ uint32_t nvfp4_scale_code(float bmax) {
  uint32_t c = f32_to_e4m3_rn_sat(bmax * 0.16666667163372040f);
  const float s = e4m3_code_to_f32(c);
  if (6.0f * s < bmax) c += 1;       // nearest was one step short of the round-up
  c = max(c, 1u);                    // floor 2^-9  (all-zero block -> code 0x01)
  return min(c, 0x7Eu);              // saturate at 448, never the NaN code
}

// Eight float32 (bf16-valued, four pairs) -> eight E2M1 codes, element 0 in bits [0,4).
__device__ __forceinline__ uint32_t nvfp4_quantize8(const float2* x, float s, float r) {
  float2 q[4];
  const float2 r2 = make_float2(r, r), ns2 = make_float2(-s, -s);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 q0 = __fmul2_rn(x[i], r2);
    const float2 e = __ffma2_rn(ns2, q0, x[i]);
    q[i] = __ffma2_rn(e, r2, q0);
  }
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(out)
      : "f"(q[0].x), "f"(q[0].y), "f"(q[1].x), "f"(q[1].y), "f"(q[2].x), "f"(q[2].y), "f"(q[3].x), "f"(q[3].y));
  // No sign fix-up is needed here: the quotient is zero only for x = +-0, and for x = -0 the two
  // refinement FMAs already turn it into +0 (e = (-s)(-0) + (-0) = +0, q = (+0) r + (-0) = +0), which is
  // what the reference's sign(x/s) * |q| gives; a negative x that merely rounds to zero keeps its sign.
  return out;
}

// MXFP8 block scale byte (exponent + 127) from the block's absolute maximum (bf16-valued).
__device__ __forceinline__ uint32_t mxfp8_scale_code(float bmax) {
  const uint32_t u = __float_as_uint(bmax);
  const int exp = static_cast<int>(u >> 23);          // biased; sign is 0
  const int man = static_cast<int>((u >> 16) & 0x7F);  // the 7 bf16 mantissa bits
  // max = (1 + man/128) * 2^(exp-127);  448 = 1.75 * 2^8  ->  e = exp-127-8 (+1 if 1+man/128 > 1.75)
  int code = exp - 8 + (man > 96 ? 1 : 0);
  if (exp == 0) code = 1;                              // zero / subnormal max
  return static_cast<uint32_t>(max(code, 1));          // floor 2^-126
}

// Eight float32 (four pairs) -> eight E4M3 bytes (element 0 in the low byte of .x); inv = 2^-e.
// The reference multiplies the rounded magnitude by sign(x / s), so a quotient that is exactly zero must lose
// its sign while a negative one that merely rounds to zero keeps it: fl(x * inv) + (+0) does that (-0 + +0 = +0,
// every other value unchanged); x * inv is exact apart from underflow, where it rounds like the reference's x / s
// (so the product is rounded on its own, not fused with the addition).
__device__ __forceinline__ uint2 mxfp8_quantize8(const float2* x, float inv) {
  uint16_t h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // scalar _rn intrinsics: never contracted into one fused multiply-add (which would round the exact tiny
    // product straight to -0 and keep the sign)
    const float q0 = __fadd_rn(__fmul_rn(x[i].x, inv), 0.0f), q1 = __fadd_rn(__fmul_rn(x[i].y, inv), 0.0f);
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(h[i]) : "f"(q1), "f"(q0));
  }
  uint2 out;
  out.x = static_cast<uint32_t>(h[0]) | (static_cast<uint32_t>(h[1]) << 16);
  out.y = static_cast<uint32_t>(h[2]) | (static_cast<uint32_t>(h[3]) << 16);
  return out;
}

// 2^(code-127) as float32 for an E8M0 byte in [1, 254].
__device__ __forceinline__ float e8m0_to_f32(uint32_t code) { return __uint_as_float(code << 23); }

// ---- SiLU with a written-down float32 exponential -------------------------------------------
// exp(x) for the SiLU prologue, defined operation by operation so that the CPU checker can restate it
// bit for bit (a library expf is only specified to a few units in the last place): every multiply and
// add below is a separately rounded IEEE float32 operation (no fused multiply-add), in this order:
//   x  <- min(max(x, -100), 100)
//   n  <- (x * log2(e) + 1.5 * 2^23) - 1.5 * 2^23           (nearest integer, ties to even)
//   r  <- (x - n * 0.693359375) - n * (-2.12194440e-4)       (Cody-Waite split of ln 2)
//   p  <- 1 + r (1 + r (1/2 + r (1/6 + r (1/24 + r (1/120 + r (1/720 + r / 5040))))))   (Horner)
//   exp <- (p * 2^floor(n/2)) * 2^(n - floor(n/2))           (two exact scalings; overflows to +inf)
// |r| <= 0.3466, so the truncated series is within 6e-9 of e^r; the result is within ~2 ulp of exp(x).
__device__ __forceinline__ float exp_det(float x) {
  x = fminf(fmaxf(x, -100.0f), 100.0f);
  const float magic = 12582912.0f;
  const float n = __fsub_rn(__fadd_rn(__fmul_rn(x, 1.44269502162933349609375f), magic), magic);
  float r = __fsub_rn(x, __fmul_rn(n, 0.693359375f));
  r = __fsub_rn(r, __fmul_rn(n, -2.12194440e-4f));
  float p = 1.98412701138295233249664306640625e-4f;                       // 1/5040
  p = __fadd_rn(__fmul_rn(p, r), 1.388888922519981861114501953125e-3f);    // 1/720
  p = __fadd_rn(__fmul_rn(p, r), 8.3333337679505348205566406250e-3f);      // 1/120
  p = __fadd_rn(__fmul_rn(p, r), 4.16666679084300994873046875e-2f);        // 1/24
  p = __fadd_rn(__fmul_rn(p, r), 0.1666666716337203979492187500f);         // 1/6
  p = __fadd_rn(__fmul_rn(p, r), 0.5f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  const int ni = __float2int_rn(n);
  const int h = ni >> 1;
  const float s1 = __uint_as_float(static_cast<uint32_t>(h + 127) << 23);
  const float s2 = __uint_as_float(static_cast<uint32_t>(ni - h + 127) << 23);
  return __fmul_rn(__fmul_rn(p, s1), s2);
}

// The same list of operations on two values at once (packed float32x2 multiplies and adds round each element like
// their scalar forms, so the results are those of exp_det).
__device__ __forceinline__ float2 exp_det2(float2 x) {
  x.x = fminf(fmaxf(x.x, -100.0f), 100.0f);
  x.y = fminf(fmaxf(x.y, -100.0f), 100.0f);
  const float2 magic = make_float2(12582912.0f, 12582912.0f), nmagic = make_float2(-12582912.0f, -12582912.0f);
  const float2 n = __fadd2_rn(__fadd2_rn(__fmul2_rn(x, make_float2(1.44269502162933349609375f, 1.44269502162933349609375f)), magic), nmagic);
  // x - n * c == x + n * (-c): the product only changes sign
  float2 r = __fadd2_rn(x, __fmul2_rn(n, make_float2(-0.693359375f, -0.693359375f)));
  r = __fadd2_rn(r, __fmul2_rn(n, make_float2(2.12194440e-4f, 2.12194440e-4f)));
  float2 p = make_float2(1.98412701138295233249664306640625e-4f, 1.98412701138295233249664306640625e-4f);
  const float c[7] = {1.388888922519981861114501953125e-3f, 8.3333337679505348205566406250e-3f,
                      4.16666679084300994873046875e-2f, 0.1666666716337203979492187500f, 0.5f, 1.0f, 1.0f};
#pragma unroll
  for (int i = 0; i < 7; ++i) p = __fadd2_rn(__fmul2_rn(p, r), make_float2(c[i], c[i]));
  const int n0 = __float2int_rn(n.x), n1 = __float2int_rn(n.y);
  const int h0 = n0 >> 1, h1 = n1 >> 1;
  const float2 s1 = make_float2(__uint_as_float(static_cast<uint32_t>(h0 + 127) << 23),
                                __uint_as_float(static_cast<uint32_t>(h1 + 127) << 23));
  const float2 s2 = make_float2(__uint_as_float(static_cast<uint32_t>(n0 - h0 + 127) << 23),
                                __uint_as_float(static_cast<uint32_t>(n1 - h1 + 127) << 23));
  return __fmul2_rn(__fmul2_rn(p, s1), s2);
}

// SiLU(g) = g / (1 + exp(-g)), float32, IEEE division (torch.nn.functional.silu on a bf16 tensor computes in
// float32 and rounds once; the caller does that rounding).
__device__ __forceinline__ float silu_det(float g) { return __fdiv_rn(g, __fadd_rn(1.0f, exp_det(-g))); }
__device__ __forceinline__ float2 silu_det2(float2 g) {
  const float2 d = __fadd2_rn(make_float2(1.0f, 1.0f), exp_det2(make_float2(-g.x, -g.y)));
  return make_float2(__fdiv_rn(g.x, d.x), __fdiv_rn(g.y, d.y));
}

#endif  // __CUDACC__
}  // namespace plq
