// 8-bit affine KV codes ("UINT8_KC128_VT_F32": K quantised per channel over groups of 128 tokens, V per
// token), the compact form the cache keeps for everything older than the 64 sink + 2048 recent tokens.
//   stats = (lo, scale) in FP32 with scale = span == 0 ? 1 : span / 255 ;  code = rn(clamp((x - lo) / scale, 0, 255))
//   x' = bf16_rne(code * scale + lo)          (multiply, add, round: each step IEEE round-to-nearest)
// Layouts (head-major, like the reference's KvCacheView, kernels/kv_cache.cuh:10-32, :52-95):
//   src    [heads, capacity, D] bf16          codes [heads, capacity, D] uint8
//   k_stats [heads, ceil(capacity/128), D, 2]  v_stats [heads, capacity, 2]
// The reference fixes D = 256 and 4 KV heads; these kernels take any D that is a multiple of 32.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int KV_GROUP = 128;

__device__ __forceinline__ uint8_t kv_code(float x, float lo, float scale) {
  return (uint8_t)__float2uint_rn(fminf(255.f, fmaxf(0.f, __fdiv_rn(__fsub_rn(x, lo), scale))));
}

// K: one thread per channel of one (head, group); grid (groups_to_pack, heads), D threads (<= 1024)
__global__ void kv_pack_k_kernel(const __nv_bfloat16* __restrict__ src, uint8_t* __restrict__ codes,
                                 float* __restrict__ stats, int capacity, int D, int group0, int* status) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, grp = group0 + blockIdx.x, d = threadIdx.x;
  const int groups = (capacity + KV_GROUP - 1) / KV_GROUP;
  const size_t base = ((size_t)h * capacity + (size_t)grp * KV_GROUP) * D + d;
  float lo = 3.402823466e38f, hi = -3.402823466e38f;
  bool finite = true;
  for (int r = 0; r < KV_GROUP; ++r) {
    const float x = __bfloat162float(src[base + (size_t)r * D]);
    finite = finite && (fabsf(x) <= 3.4e38f);
    lo = fminf(lo, x); hi = fmaxf(hi, x);
  }
  if (!finite) { set_status(status, KID_KV, FF_ERR_NONFINITE, h, grp); lo = 0.f; hi = 0.f; }
  const float span = __fsub_rn(hi, lo), scale = span == 0.f ? 1.f : __fdiv_rn(span, 255.f);
  const size_t si = (((size_t)h * groups + grp) * D + d) * 2;
  stats[si] = lo; stats[si + 1] = scale;
  for (int r = 0; r < KV_GROUP; ++r)
    codes[base + (size_t)r * D] = kv_code(__bfloat162float(src[base + (size_t)r * D]), lo, scale);
}

// V: one warp per (head, token); grid (ceil(tokens/8), heads), 256 threads
__global__ void kv_pack_v_kernel(const __nv_bfloat16* __restrict__ src, uint8_t* __restrict__ codes,
                                 float* __restrict__ stats, int capacity, int D, int pos0, int tokens, int* status) {
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.y, t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= tokens) return;
  const int pos = pos0 + t;
  const size_t base = ((size_t)h * capacity + pos) * D;
  float lo = 3.402823466e38f, hi = -3.402823466e38f;
  bool finite = true;
  for (int d = lane; d < D; d += 32) {
    const float x = __bfloat162float(src[base + d]);
    finite = finite && (fabsf(x) <= 3.4e38f);
    lo = fminf(lo, x); hi = fmaxf(hi, x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o)); }
  if (!__all_sync(0xffffffffu, finite)) { if (lane == 0) set_status(status, KID_KV, FF_ERR_NONFINITE, h, pos); lo = 0.f; hi = 0.f; }
  const float span = __fsub_rn(hi, lo), scale = span == 0.f ? 1.f : __fdiv_rn(span, 255.f);
  if (lane == 0) { stats[((size_t)h * capacity + pos) * 2] = lo; stats[((size_t)h * capacity + pos) * 2 + 1] = scale; }
  for (int d = lane; d < D; d += 32) codes[base + d] = kv_code(__bfloat162float(src[base + d]), lo, scale);
}

// codes -> bf16 for tokens [pos0, pos0 + tokens); is_k selects the statistics layout
__global__ void kv_unpack_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ stats,
                                 __nv_bfloat16* __restrict__ dst, int capacity, int D, int heads, int pos0, int tokens,
                                 int is_k) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)heads * tokens * D) return;
  const int d = (int)(i % D), t = (int)((i / D) % tokens), h = (int)(i / ((size_t)D * tokens));
  const int pos = pos0 + t;
  const size_t at = ((size_t)h * capacity + pos) * D + d;
  const int groups = (capacity + KV_GROUP - 1) / KV_GROUP;
  const size_t si = is_k ? (((size_t)h * groups + pos / KV_GROUP) * D + d) * 2 : ((size_t)h * capacity + pos) * 2;
  dst[at] = __float2bfloat16_rn(__fadd_rn(__fmul_rn((float)codes[at], stats[si + 1]), stats[si]));
}

}  // namespace ff
using namespace ff;

// Pack K groups [group0, group0 + groups) (128 tokens each, per-channel statistics).
FF_EXPORT int ff_kv_pack_k(const void* src, void* codes, float* stats, int heads, int capacity, int D, int group0,
                           int groups, int* status, cudaStream_t s) {
  if (heads <= 0 || capacity <= 0 || D <= 0 || D > 1024 || D % 32 || groups <= 0 || group0 < 0) return FF_HOST_BAD_SHAPE;
  if ((long long)(group0 + groups) * KV_GROUP > capacity) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(kv_pack_k_kernel, dim3(groups, heads), dim3(D), 0, s, 0, (const __nv_bfloat16*)src, (uint8_t*)codes,
                          stats, capacity, D, group0, status)) return lr;
  return launch_result();
}

// Pack V tokens [pos0, pos0 + tokens) (per-token statistics).
FF_EXPORT int ff_kv_pack_v(const void* src, void* codes, float* stats, int heads, int capacity, int D, int pos0, int tokens,
                           int* status, cudaStream_t s) {
  if (heads <= 0 || capacity <= 0 || D <= 0 || D % 32 || tokens <= 0 || pos0 < 0 || pos0 + tokens > capacity) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(kv_pack_v_kernel, dim3((tokens + 7) / 8, heads), dim3(256), 0, s, 0, (const __nv_bfloat16*)src,
                          (uint8_t*)codes, stats, capacity, D, pos0, tokens, status)) return lr;
  return launch_result();
}

FF_EXPORT int ff_kv_unpack(const void* codes, const float* stats, void* dst, int heads, int capacity, int D, int pos0,
                           int tokens, int is_k, cudaStream_t s) {
  if (heads <= 0 || capacity <= 0 || D <= 0 || tokens <= 0 || pos0 < 0 || pos0 + tokens > capacity) return FF_HOST_BAD_SHAPE;
  const size_t total = (size_t)heads * tokens * D;
  if (int lr = launch_pdl(kv_unpack_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, (const uint8_t*)codes, stats,
                          (__nv_bfloat16*)dst, capacity, D, heads, pos0, tokens, is_k)) return lr;
  return launch_result();
}
