// Shared pieces of the tcgen05 kernels (fused GEMM and tensor-core GEMV): tile constants, shared-memory
// and instruction descriptors, tensor-map builders.
#pragma once

#include <cuda.h>

#include "plq_common.cuh"

namespace plq {

constexpr int kBM = 128;                          // rows of the M-side operand per CTA and MMA
constexpr int kStageKBytes = 128;                 // bytes of K per row per stage (one swizzle span)
constexpr int kABytes = kBM * kStageKBytes;       // 16 KiB
constexpr int kSfChunk = 512;                     // one tiled scale chunk: 128 rows x 4 scales

// Tensor maps: code matrices as 2-D u8 [rows, row bytes] with 128-byte swizzled boxes; tiled
// scale buffers as 3-D int32 [128 words = one 512-byte chunk, chunks per group, 128-row groups].
struct GemmMaps {
  CUtensorMap a_lo, b_lo, a_hi, b_hi, sfa_lo, sfb_lo, sfa_hi, sfb_hi;
};

// Shared-memory matrix descriptors, split into a low word (address field, changes per stage) and a
// constant high word.
//   K-major tile of 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart:
//     low  = start address >> 4 | leading byte offset 1 (unused for swizzled K-major) at bit 16
//     high = stride byte offset 1024 >> 4 | descriptor version 1 at bit 46 | SWIZZLE_128B (2) at bit 61
//   one 512-byte scale chunk, 32 rows x 16 bytes, no swizzle, 8-row groups 128 bytes apart:
//     low  = start address >> 4;   high = stride byte offset 128 >> 4 | version 1 at bit 46
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t kDescHiSf = (128u >> 4) | (1u << 14);
__device__ __forceinline__ uint32_t desc_lo_sw128(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_sf(uint32_t saddr) { return (saddr & 0x3FFFFu) >> 4; }
// Instruction descriptor of a block-scaled MMA (K-major operands).
//   [4,6) B scale id  [7,10) A format  [10,13) B format  [17,23) N/8  [23] scale format
//   [24,29) M/16  [29,31) A scale id
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t m, uint32_t n, uint32_t scale_is_e8m0) {
  return (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | (scale_is_e8m0 << 23) | ((m >> 4) << 24);
}

// Host side (defined in plq_gemm.cu).
// u8 matrix [rows, row_bytes], box = 128 bytes x box_rows, 128-byte swizzle, zero fill out of bounds.
int make_tmap(CUtensorMap* tm, const void* base, int64_t rows, int64_t row_bytes, int box_rows);
// Tiled scale buffer as int32 [128 words, chunks per group, groups]; box = 4 chunks of `box_groups` groups.
int make_sf_tmap(CUtensorMap* tm, const void* base, int64_t chunks, int64_t groups, int box_groups);

}  // namespace plq
