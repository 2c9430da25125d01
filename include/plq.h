/*
 * plq.h - C ABI of libplq_b200.so: the mixed NVFP4 / MXFP8 quantised-linear hot path on B200.
 *
 * Every entry point takes raw device pointers, 64-bit sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*; NULL = the legacy default stream), launches
 * asynchronously on that stream and returns an int status: 0 = ok, negative = argument or
 * host-side error detected before anything was launched (see plq_status_string), positive
 * values are only ever written by a kernel into the caller's status word.  The caller owns
 * and allocates every buffer, outputs and workspaces included; the library never allocates
 * or frees device memory (plq_gemv_static_scratch uses an array built into the library image
 * instead of a caller's workspace).  There is no CPU fallback: on a device that is not sm_100
 * the calls return PLQ_ERR_ARCH.
 *
 * Packed operand ("rows x K" matrix whose last K_hi columns are the outlier subspace):
 *   lo_codes  u8 [rows, K_lo/2]   E2M1, two per byte, low nibble = lower K
 *   lo_sf     u8                  E4M3 scale per 16 elements
 *   hi_codes  u8 [rows, K_hi]     E4M3
 *   hi_sf     u8                  E8M0 scale (exponent + 127) per 32 elements
 * Scale buffers come in two layouts:
 *   PLQ_SF_ROWMAJOR  [rows, K_lo/16] and [rows, K_hi/32]  (the reference spec's layout,
 *                    docs/specs/spec-mxfp8-nvfp4.md:163-169)
 *   PLQ_SF_TILED     512-byte chunks of 128 rows x 4 scales, byte (r%32)*16 + (r%128)/32*4
 *                    + (k%4), chunks ordered K-fastest, rows and scales padded to 128 and 4:
 *                    the order a block-scaled tcgen05.mma reads from tensor memory.
 *                    Size in bytes: plq_sf_tiled_bytes(rows, n_scales_per_row).  The pack kernels
 *                    write only the real entries.  Padding scales beyond the row's last one (inside
 *                    its last chunk of four) must be zero: the MMA multiplies them with zero codes,
 *                    and 0 x NaN is NaN.  Padding rows may hold anything: they only scale output rows
 *                    that are never stored.
 * Constraints: K_lo % 64 == 0, K_hi % 32 == 0, K % 128 == 0 when a Hadamard rotation or
 * RMSNorm is requested, K <= 32768; all pointers 16-byte aligned.
 *
 * Reference interfaces these replace are cited per function as path:line inside the
 * reference project (Ther-LF/plaquant).
 */
#ifndef PLQ_H_
#define PLQ_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define PLQ_API __attribute__((visibility("default")))
#else
#define PLQ_API
#endif

#define PLQ_OK              0
#define PLQ_ERR_NULL       -1   /* a required pointer is NULL */
#define PLQ_ERR_SHAPE      -2   /* a size violates the constraints above */
#define PLQ_ERR_ALIGN      -3   /* a pointer is not 16-byte aligned */
#define PLQ_ERR_ARCH       -4   /* current device is not compute capability 10.x */
#define PLQ_ERR_CUDA       -5   /* a CUDA runtime call failed (plq_last_cuda_error) */
#define PLQ_ERR_TENSORMAP  -6   /* cuTensorMapEncodeTiled rejected a descriptor */
#define PLQ_ERR_LIMIT      -7   /* size beyond a documented maximum */
#define PLQ_DEV_TIMEOUT     1   /* written by a kernel: a bounded wait ran out */
#define PLQ_DEV_PROTOCOL    2   /* written by a kernel: a fused reduction was called on the wrong buffer set */
#define PLQ_DEV_RANGE       3   /* written by a kernel: a cache position read from device memory was out of range */

#define PLQ_SF_ROWMAJOR 0
#define PLQ_SF_TILED    1

/* Library / ABI version (major * 100 + minor). */
PLQ_API int plq_version(void);

/* Human-readable text for a status value.  Never NULL. */
PLQ_API const char* plq_status_string(int status);

/* cudaError_t of the last failing runtime call on this thread (0 if none). */
PLQ_API int plq_last_cuda_error(void);

/* 0 if the current device can run the kernels (compute capability 10.x), else PLQ_ERR_ARCH. */
PLQ_API int plq_device_check(void);

/* Bytes of a PLQ_SF_TILED buffer for `rows` rows and `n_sf` scales per row. */
PLQ_API int64_t plq_sf_tiled_bytes(int64_t rows, int64_t n_sf);

/*
 * Quantise-and-pack a bf16 matrix x[rows, k] (row stride k): optional block-Hadamard(128)
 * rotation of every 128-column block (y = bf16((x.float() @ H128)/..)), then the last k_hi
 * columns go to MXFP8 and the rest to NVFP4.
 * Replaces, for activations: ActQuantizer.forward FP branch, promix/quantize/quant_utils.py:182-224
 * (fake_quantize_nvfp4 :710-751, fake_quantize_mxfp8 :660-707) preceded by the online Hadamard
 * of inference/quantize.py:447-448 / inference/forward_pass.py:283-284.
 * For weights (x = W[N, K]): WeightQuantizer round-to-nearest, promix/quantize/kv_quant.py:161-166,
 * after _apply_had_to_linear, promix/quantize/rotation.py:100-116.
 */
PLQ_API int plq_pack(const void* x_bf16, int64_t rows, int64_t k, int64_t k_hi, int hadamard,
             void* lo_codes, void* lo_sf, void* hi_codes, void* hi_sf, int sf_layout,
             void* stream);

/*
 * Fused RMSNorm -> [block-Hadamard(128)] -> quantise-and-pack of hidden states x[rows, k]:
 *   y = bf16(gamma * (x * rsqrt(mean(x^2) + eps))), float32 arithmetic,
 * then as plq_pack.  Replaces rms_norm, inference/forward_pass.py:33-39, followed by the
 * activation quantiser of the next linear (forward_pass.py:191-196, 264-268).
 */
PLQ_API int plq_rmsnorm_pack(const void* x_bf16, const void* gamma_bf16, float eps,
                     int64_t rows, int64_t k, int64_t k_hi, int hadamard,
                     void* lo_codes, void* lo_sf, void* hi_codes, void* hi_sf, int sf_layout,
                     void* stream);

/*
 * plq_pack fused with the element-wise step that produces its input in the decoder's MLP:
 * quantises bf16(bf16(SiLU(gate)) * up), gate and up being bf16 [rows, k] with row stride `ld`
 * elements (ld % 8 == 0; the two halves of one gate_up output: up = gate + k).  Both roundings of
 * the two PyTorch ops it replaces are kept.  Replaces `F.silu(gate) * up` followed by the
 * rotation + quantiser of down_proj, inference/forward_pass.py:266-269.
 */
PLQ_API int plq_silu_mul_pack(const void* gate_bf16, const void* up_bf16, int64_t ld, int64_t rows, int64_t k,
                              int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf, void* hi_codes,
                              void* hi_sf, int sf_layout, void* stream);

/*
 * plq_rmsnorm_pack fused with the residual add in front of it: h = bf16(residual + x) (one rounding,
 * as torch's bf16 add) is written to h_out_bf16 [rows, k] (may alias residual_bf16 or x_bf16) and
 * then normalised, rotated and quantised.  Replaces `x = residual + attn_out; x = rms_norm(x, ln2)`
 * and the quantiser of the next linear, inference/forward_pass.py:258-264.
 */
PLQ_API int plq_add_rmsnorm_pack(const void* x_bf16, const void* residual_bf16, void* h_out_bf16,
                                 const void* gamma_bf16, float eps, int64_t rows, int64_t k, int64_t k_hi,
                                 int hadamard, void* lo_codes, void* lo_sf, void* hi_codes, void* hi_sf,
                                 int sf_layout, void* stream);

/*
 * Tensor-parallel form of plq_add_rmsnorm_pack: the all-reduce that follows a row-parallel linear, the residual
 * add, the RMSNorm and the quantiser of the next linear in one kernel.  x = bf16(sum over the ranks of their
 * partial outputs), summed in float32 in rank order so that every rank gets the same bits; the partial outputs
 * are read from the ranks' own buffers over NVLink (peer loads; no library collective, no multicast).
 *   peer_x_dev      device array [world] of addresses: rank r's bf16 [rows, k] buffer (this rank's own included),
 *                   each written by the kernel that precedes this call in rank r's stream
 *   peer_flags_dev  device array [world] of addresses: rank r's int32 flags[world]
 *   flags, sync     this rank's flags[world] and int32 sync[2], zero before the first call, owned by the library
 *                   afterwards
 *   buffer_index    which of the caller's two sets of x buffers `peer_x_dev` names (0 or 1; -1 = not checked)
 * Every rank must make the same sequence of calls, and consecutive calls must alternate between two sets of x
 * buffers, starting with set 0: a rank may be one call ahead of a peer that is still reading, and it is the
 * alternation alone (no other collective is needed in between) that keeps it from overwriting what the peer
 * reads - rank r writes set b again only after its call in between has seen every peer announce that call,
 * i.e. after every peer has finished the earlier call on set b.  The kernel numbers the calls itself (in
 * `sync`); call c must use set (c + 1) % 2, counting from c = 1.  A CUDA graph that is replayed must therefore
 * contain an even number of these calls, or a replay would reuse the set of the call just before it: the kernel
 * checks `buffer_index` against its own count and stores PLQ_DEV_PROTOCOL to `dev_status` on a mismatch (the
 * output is then void).  A rank that does not show up within the bounded wait makes the others store
 * PLQ_DEV_TIMEOUT to `dev_status` and finish (their output is then void).
 * Replaces `dist.all_reduce` + `x = residual + x; x = rms_norm(x, ...)` + the next quantiser in a
 * tensor-parallel decoder layer (inference/forward_pass.py:258-264 under tensor parallelism).
 */
PLQ_API int plq_allreduce_add_rmsnorm_pack(const void* const* peer_x_dev, void* const* peer_flags_dev, int32_t* flags,
                                           int32_t* sync, int world, int rank, int buffer_index,
                                           const void* residual_bf16,
                                           void* h_out_bf16, const void* gamma_bf16, float eps, int64_t rows,
                                           int64_t k, int64_t k_hi, int hadamard, void* lo_codes, void* lo_sf,
                                           void* hi_codes, void* hi_sf, int sf_layout, int32_t* dev_status,
                                           void* stream);

/*
 * Scattered form of plq_allreduce_add_rmsnorm_pack for prefill batches (sequence-parallel between the row-parallel
 * linear and the next column-parallel one): a reduce-scatter of the partial outputs, the residual add and RMSNorm
 * on this rank's rows only, and an all-gather of the PACKED rows (4.5 bits per element instead of 16) in one
 * kernel.  The ranks' partial outputs are bf16 [total_rows, k]; this rank handles rows [row0, row0 + rows).
 *   peer_x_dev       as above, the buffers being [total_rows, k]
 *   out_tbl_dev      device array [32] of addresses: entry 8 * i + r is rank r's buffer of output i (0 lo_codes
 *                    [total_rows, k_lo/2], 1 lo_sf ROW-MAJOR [total_rows, k_lo/16], 2 hi_codes [total_rows, k_hi],
 *                    3 hi_sf ROW-MAJOR [total_rows, k_hi/32]); the rows are stored at their global row index into
 *                    every rank's buffers by peer stores, whole 128-byte lines per warp
 *   residual, h_out  this rank's slice [rows, k] of the residual stream (local memory)
 *   lo_codes, lo_sf_rowmajor, hi_codes, hi_sf_rowmajor   this rank's own buffers (column `rank` of the table)
 *   lo_sf_tiled, hi_sf_tiled   local buffers of plq_sf_tiled_bytes(total_rows, ...) bytes, or both NULL: when
 *                    given, a second small kernel rewrites the gathered scale bytes of ALL rows into the tiled
 *                    layout the GEMM reads (padding written as zero)
 *   flags            int32 [64]: words [0, world) announce a call, words [32, 32 + world) its completion
 * The first kernel completes only after every rank has stored its rows everywhere and said so (bounded wait,
 * PLQ_DEV_TIMEOUT otherwise): when the call's work has completed on the stream, the packed buffers hold all
 * `total_rows` rows and no peer reads this rank's partial outputs of this call any more.  Call sequence, buffer
 * alternation and `buffer_index` as for plq_allreduce_add_rmsnorm_pack (the output buffers alternate together
 * with the partial-output buffers).  Every rank must call with rows >= 1.
 * Replaces `dist.all_reduce` + residual add + rms_norm + quantiser for prefill batches of a tensor-parallel
 * decoder layer (inference/forward_pass.py:258-264 under tensor parallelism); the reference has no such step.
 */
PLQ_API int plq_reduce_scatter_add_rmsnorm_pack(const void* const* peer_x_dev, void* const* peer_flags_dev,
                                                int32_t* flags, int32_t* sync, int world, int rank, int buffer_index,
                                                void* const* out_tbl_dev, int64_t row0, int64_t total_rows,
                                                const void* residual_bf16, void* h_out_bf16, const void* gamma_bf16,
                                                float eps, int64_t rows, int64_t k, int64_t k_hi, int hadamard,
                                                void* lo_codes, void* lo_sf_rowmajor, void* hi_codes,
                                                void* hi_sf_rowmajor, void* lo_sf_tiled, void* hi_sf_tiled,
                                                int32_t* dev_status, void* stream);

/*
 * Rotary position embedding of the query and key heads of a fused QKV projection and the append of keys and values
 * to the cache, one pass.  qkv: bf16 [batch * t, ld], each row [heads | kv_heads | kv_heads] x head_dim (128);
 * cos, sin: float32 [t, 128], row i for the i-th new position.  Per head, x1 = first half, x2 = second half, every
 * operation rounded to float32 on its own, one rounding to bf16:
 *     out[i] = x1[i] * cos[i] - x2[i] * sin[i],   out[64 + i] = x2[i] * cos[64 + i] + x1[i] * sin[64 + i].
 * Outputs: q_out bf16 [batch * t, heads, 128]; rotated keys and unchanged values go to k_cache / v_cache, bf16
 * [batch, t_max, kv_heads, 128], at positions pos .. pos + t - 1, where pos is read from `pos_dev` (a device
 * scalar, so that a decode step replayed from a CUDA graph appends at the current position) or, with pos_dev
 * NULL, is the argument `pos`.  A position outside [0, t_max) read from device memory stores nothing and writes
 * PLQ_DEV_RANGE to `dev_status`.
 * Replaces apply_rotary_pos_emb and the cache update of the reference's decoder layer
 * (inference/forward_pass.py:82-110, 216-247), which run as a dozen PyTorch kernels; the arithmetic is that of
 * `x.float() * cos + rotate_half(x).float() * sin` rounded to bf16.
 */
PLQ_API int plq_rope_kv_append(const void* qkv_bf16, int64_t ld, const void* cos_f32, const void* sin_f32,
                               int64_t batch, int64_t t, int64_t heads, int64_t kv_heads, int64_t head_dim,
                               void* q_out_bf16, void* k_cache_bf16, void* v_cache_bf16, int64_t t_max,
                               const int64_t* pos_dev, int64_t pos, int32_t* dev_status, void* stream);

/*
 * One column block of GPTQ for the block-scaled formats: columns [col0, col0 + count), count <= 128, of the
 * float32 weight w[rows, k] (which already carries the corrections of the earlier blocks) are rounded one after
 * the other - each against the block scale frozen beforehand (`lo_sf` [rows, (k - k_hi)/16] E4M3 bytes for the
 * NVFP4 columns, `hi_sf` [rows, k_hi/32] E8M0 bytes for the last k_hi, both row-major) - and the rounding error of
 * column i, divided by hinv[i, i], is folded into the later columns of the block with row i of `hinv` (the upper
 * Cholesky factor of the inverse Hessian, [k, k]).  Outputs: q[rows, k] receives the dequantised values of the
 * block's columns, err[rows, count] the scaled errors (the caller applies them to the columns behind the block:
 * w[:, col0 + count:] -= err @ hinv[col0 : col0 + count, col0 + count:]), codes[rows, k] one code per element.
 * `w` itself is not modified.
 * Replaces the per-column inner loop of GPTQ.fasterquant with quantize_column_with_frozen_scale,
 * promix/quantize/gptq.py:142-205 and promix/quantize/quant_utils.py:616-657.
 */
PLQ_API int plq_gptq_block_frozen(const void* w_f32, int64_t ldw, const void* hinv_f32, int64_t ldh,
                                  const void* lo_sf, const void* hi_sf, int64_t rows, int64_t k, int64_t k_hi,
                                  int64_t col0, int64_t count, void* q_f32, int64_t ldq, void* err_f32,
                                  void* codes_u8, void* stream);

/*
 * Dequantise a packed matrix back to bf16 [rows, k_lo + k_hi] (= the fake quantiser's return
 * value, promix/quantize/quant_utils.py:750-751, :706-707).
 */
PLQ_API int plq_unpack(const void* lo_codes, const void* lo_sf, const void* hi_codes, const void* hi_sf,
               int sf_layout, int64_t rows, int64_t k_lo, int64_t k_hi, void* y_bf16,
               void* stream);

/*
 * Fused mixed GEMM: y[m, n] (bf16, row stride ldy elements) = deq(A)[m, :] . deq(B)[n, :]
 * with A = packed activations (m rows), B = packed weights (n rows), both K-major, scale
 * buffers in PLQ_SF_TILED layout.  One kernel, one tensor-memory accumulator: the NVFP4
 * K-range runs as tcgen05.mma kind::mxf4nvf4 and the MXFP8 K-range as kind::mxf8f6f4 on top.
 * `dev_status` is a device int32 the kernel sets to PLQ_DEV_TIMEOUT if a bounded wait ran
 * out (the output is then undefined); it must be zero on entry and may not be NULL.
 * Replaces the quantised linear itself, promix/quantize/quant_utils.py:389 /
 * inference/forward_pass.py:319, in the two-K-phase call shape of fused_mixed_gemm,
 * kernels/mixed_gemm/mixed_gemm.cu:346-350.
 */
PLQ_API int plq_mixed_gemm(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                   const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                   int64_t m, int64_t n, int64_t k_lo, int64_t k_hi,
                   void* y_bf16, int64_t ldy, int32_t* dev_status, void* stream);

/*
 * plq_mixed_gemm with the tile shape chosen by the caller instead of by the built-in heuristic
 * (tests and tuning).  Same reference counterpart.
 */
#define PLQ_GEMM_AUTO          0
#define PLQ_GEMM_128x128       1   /* one CTA per 128 x 128 tile, two accumulator stages */
#define PLQ_GEMM_128x256       2   /* one CTA per 128 x 256 tile */
#define PLQ_GEMM_PAIR_256x256  3   /* a CTA pair per 256 x 256 tile (tcgen05.mma.cta_group::2) */
PLQ_API int plq_mixed_gemm_variant(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                                   const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                                   int64_t m, int64_t n, int64_t k_lo, int64_t k_hi,
                                   void* y_bf16, int64_t ldy, int32_t* dev_status, void* stream, int variant);

/*
 * Decode GEMV, m <= 8: same contract as plq_mixed_gemm but streaming the weights once from
 * HBM; scale buffers of both operands in PLQ_SF_ROWMAJOR layout.
 * `workspace` (device memory, 16-byte aligned, at least plq_gemv_workspace_bytes(n) bytes, zeroed
 * once by the caller and left zeroed by every call) lets the kernel cut K into slices whose
 * partial sums it combines in a fixed order; calls that share a workspace must not overlap on
 * the GPU.  With workspace == NULL only shapes that need no K slicing are accepted.
 */
PLQ_API int64_t plq_gemv_workspace_bytes(int64_t n);
PLQ_API int plq_gemv(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
             const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
             int64_t m, int64_t n, int64_t k_lo, int64_t k_hi,
             void* y_bf16, int64_t ldy, void* workspace, int64_t workspace_bytes, void* stream);

/*
 * plq_gemv for callers that cannot supply a workspace (no counterpart in the reference).
 * Meant for hosts that are unable to allocate device memory on the library's behalf: a serving
 * process that has already claimed all of HBM for its own pool, or a plugin interface that passes
 * inputs and outputs and nothing else.  Inputs, outputs and results are exactly those of plq_gemv;
 * the K-slice scratch is an ~8.4 MB array built into the library image (resident on every GPU
 * that loads the library, until the process exits), which limits this entry point to
 * n <= 32768 output features: larger n returns PLQ_ERR_LIMIT.  The call allocates and frees
 * nothing.  The first call on each device looks up the array's device address and zeroes its
 * ticket area (after all argument checks have passed); make that first call before any stream
 * capture.  Host threads may make it concurrently: they resolve the same address, which is
 * published atomically.  All calls on a device share the
 * one array (it keeps the previous call's partial sums, which the next call overwrites before
 * reading): calls that overlap on the GPU, e.g. on two streams, race and must be serialised by
 * the caller.
 */
PLQ_API int plq_gemv_static_scratch(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes,
                                    const void* a_hi_sf, const void* b_lo_codes, const void* b_lo_sf,
                                    const void* b_hi_codes, const void* b_hi_sf, int64_t m, int64_t n,
                                    int64_t k_lo, int64_t k_hi, void* y_bf16, int64_t ldy, void* stream);

/*
 * Decode GEMV on the tensor cores, m <= 16: same operands and scale layout as plq_mixed_gemm
 * (A = packed activations, B = packed weights, both with PLQ_SF_TILED scale buffers), same result
 * contract.  The weight rows are the 128-row side of the block-scaled tcgen05.mma and the m
 * activation rows the narrow side (N = 16 of the instruction), so the packed weights stream HBM -> shared memory -> tensor core
 * untouched by any thread.  When n gives fewer 128-row tiles than SMs, a thread-block cluster of up
 * to 8 CTAs shares each tile along K and combines the partial sums through distributed shared
 * memory in a fixed order; no scratch memory is needed and results do not depend on timing.
 * The kernel is launched with programmatic stream serialisation: its set-up may run while the
 * previous kernel of the stream drains; it waits for that kernel's completion before it reads an
 * operand or writes y.  With PLQ_GEMV_STATIC_B in `flags` the caller promises that the B operand
 * (weight codes and scales) was complete before the kernels that precede this call in the stream
 * were launched - true for weights packed at load time, not for a weight packed by the call just
 * before - and the first weight loads are issued before that wait (about 10 % on the largest
 * decode shape).  `dev_status` as for plq_mixed_gemm.
 * Replaces the same reference lines as plq_gemv (the quantised linear at decode batch sizes,
 * promix/quantize/quant_utils.py:389 / inference/forward_pass.py:319).
 */
#define PLQ_GEMV_STATIC_B 1   /* flags: the B operand is never written by the kernels just before the call */
PLQ_API int plq_gemv_tc(const void* a_lo_codes, const void* a_lo_sf, const void* a_hi_codes, const void* a_hi_sf,
                        const void* b_lo_codes, const void* b_lo_sf, const void* b_hi_codes, const void* b_hi_sf,
                        int64_t m, int64_t n, int64_t k_lo, int64_t k_hi,
                        void* y_bf16, int64_t ldy, int32_t* dev_status, int flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PLQ_H_ */
