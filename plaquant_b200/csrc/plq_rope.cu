// Rotary position embedding of the query and key heads of a fused QKV projection and the append of the keys and
// values to the cache, in one pass over the projection's output (inference/forward_pass.py:82-110 and 216-247 in
// the reference: apply_rotary_pos_emb, then the cache update).  HBM-bound: every element of [rows, (h + 2 kv) * 128]
// is read once and written once.
//
// Arithmetic, per element pair (x1 = element i of the head's first half, x2 = element i of its second half), in
// float32 with every operation rounded on its own (no fused multiply-add), then one rounding to bf16:
//     out[i]      = x1 * cos[i]      + (-x2) * sin[i]
//     out[64 + i] = x2 * cos[64 + i] +   x1  * sin[64 + i]
// which is `x.float() * cos + rotate_half(x).float() * sin` of the PyTorch formulation, bit for bit.
#include "plq_common.cuh"

namespace plq {

constexpr int kRopeHeadDim = 128;

struct RopeArgs {
  const uint4* qkv;        // bf16 [rows, ld]: [q heads | k heads | v heads] per row
  const float* cos;        // float32 [t, 128]: row tt belongs to position pos + tt
  const float* sin;
  uint4* q_out;            // bf16 [rows, heads, 128]
  uint4* k_dst;            // bf16 [batch, t_max, kv_heads, 128]
  uint4* v_dst;
  const long long* pos_dev;  // device scalar: first cache position of this call, or nullptr to use `pos`
  long long pos, t_max;
  int* status;
  long long ld8;           // row stride of qkv in 16-byte units
  long long total;         // rows * (heads + 2 kv_heads) * 8 threads
  int t, heads, kv_heads;
};

__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__global__ void __launch_bounds__(256, 6) rope_kv_append_kernel(const RopeArgs a) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= a.total) return;
  const int all_heads = a.heads + 2 * a.kv_heads;
  const int j = static_cast<int>(idx & 7);                              // which 8 elements of each half
  const int head = static_cast<int>((idx >> 3) % all_heads);
  const long long row = (idx >> 3) / all_heads;
  const long long b = row / a.t;
  const int tt = static_cast<int>(row - b * a.t);
  const uint4* src = a.qkv + row * a.ld8 + static_cast<long long>(head) * 16 + j;
  uint4 lo = src[0], hi = src[8];
  if (head < a.heads + a.kv_heads) {
    float x1[8], x2[8];
    unpack_bf16x8(lo, x1);
    unpack_bf16x8(hi, x2);
    const float4* c1 = reinterpret_cast<const float4*>(a.cos + static_cast<size_t>(tt) * kRopeHeadDim + 8 * j);
    const float4* s1 = reinterpret_cast<const float4*>(a.sin + static_cast<size_t>(tt) * kRopeHeadDim + 8 * j);
    const float4 ca = c1[0], cb = c1[1], cc = c1[16], cd = c1[17];      // cos[8j..8j+7], cos[64+8j..]
    const float4 sa = s1[0], sb = s1[1], sc = s1[16], sd = s1[17];
    const float cl[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float ch[8] = {cc.x, cc.y, cc.z, cc.w, cd.x, cd.y, cd.z, cd.w};
    const float sl[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    const float sh[8] = {sc.x, sc.y, sc.z, sc.w, sd.x, sd.y, sd.z, sd.w};
    float o1[8], o2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o1[i] = __fadd_rn(__fmul_rn(x1[i], cl[i]), __fmul_rn(-x2[i], sl[i]));
      o2[i] = __fadd_rn(__fmul_rn(x2[i], ch[i]), __fmul_rn(x1[i], sh[i]));
    }
    lo = make_uint4(pack_bf16x2(o1[0], o1[1]), pack_bf16x2(o1[2], o1[3]), pack_bf16x2(o1[4], o1[5]), pack_bf16x2(o1[6], o1[7]));
    hi = make_uint4(pack_bf16x2(o2[0], o2[1]), pack_bf16x2(o2[2], o2[3]), pack_bf16x2(o2[4], o2[5]), pack_bf16x2(o2[6], o2[7]));
  }
  uint4* dst;
  if (head < a.heads) {
    dst = a.q_out + (row * a.heads + head) * 16 + j;
  } else {
    const long long p = (a.pos_dev != nullptr ? *a.pos_dev : a.pos) + tt;
    if (p < 0 || p >= a.t_max) {                     // the cache is full: nothing is stored, the caller is told
      if (a.status != nullptr) atomicExch(a.status, PLQ_DEV_RANGE);
      return;
    }
    const bool is_k = head < a.heads + a.kv_heads;
    const int kh = head - a.heads - (is_k ? 0 : a.kv_heads);
    dst = (is_k ? a.k_dst : a.v_dst) + ((b * a.t_max + p) * a.kv_heads + kh) * 16 + j;
  }
  dst[0] = lo;
  dst[8] = hi;
}

}  // namespace plq

extern "C" int plq_rope_kv_append(const void* qkv_bf16, int64_t ld, const void* cos_f32, const void* sin_f32,
                                  int64_t batch, int64_t t, int64_t heads, int64_t kv_heads, int64_t head_dim,
                                  void* q_out_bf16, void* k_cache_bf16, void* v_cache_bf16, int64_t t_max,
                                  const int64_t* pos_dev, int64_t pos, int32_t* dev_status, void* stream) {
  using namespace plq;
  if (head_dim != kRopeHeadDim) return PLQ_ERR_SHAPE;
  if (batch < 1 || t < 1 || heads < 1 || kv_heads < 1 || t_max < 1) return PLQ_ERR_SHAPE;
  if (ld < (heads + 2 * kv_heads) * kRopeHeadDim || ld % 8 != 0) return PLQ_ERR_SHAPE;
  if (pos_dev == nullptr && (pos < 0 || pos + t > t_max)) return PLQ_ERR_SHAPE;
  if (batch * t > 0x7FFFFFFF || heads + 2 * kv_heads > 4096) return PLQ_ERR_LIMIT;
  if (!qkv_bf16 || !cos_f32 || !sin_f32 || !q_out_bf16 || !k_cache_bf16 || !v_cache_bf16) return PLQ_ERR_NULL;
  if (!aligned16(qkv_bf16) || !aligned16(cos_f32) || !aligned16(sin_f32) || !aligned16(q_out_bf16) ||
      !aligned16(k_cache_bf16) || !aligned16(v_cache_bf16))
    return PLQ_ERR_ALIGN;
  int st = device_check();
  if (st != PLQ_OK) return st;
  RopeArgs a;
  a.qkv = static_cast<const uint4*>(qkv_bf16);
  a.cos = static_cast<const float*>(cos_f32);
  a.sin = static_cast<const float*>(sin_f32);
  a.q_out = static_cast<uint4*>(q_out_bf16);
  a.k_dst = static_cast<uint4*>(k_cache_bf16);
  a.v_dst = static_cast<uint4*>(v_cache_bf16);
  a.pos_dev = reinterpret_cast<const long long*>(pos_dev);
  a.pos = pos;
  a.t_max = t_max;
  a.status = dev_status;
  a.ld8 = ld / 8;
  a.total = batch * t * (heads + 2 * kv_heads) * 8;
  a.t = static_cast<int>(t);
  a.heads = static_cast<int>(heads);
  a.kv_heads = static_cast<int>(kv_heads);
  const long long blocks = (a.total + 255) / 256;
  rope_kv_append_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  PLQ_CUDA_TRY(cudaGetLastError());
  return PLQ_OK;
}
