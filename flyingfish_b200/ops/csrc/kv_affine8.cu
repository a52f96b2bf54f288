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
#include "mma_sync.cuh"

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


// ---------------------------------------------------------------------------------------------------------------
// Paged compact store. The engine seals whole 128-token groups of a sequence that have left the recent window: the
// two BF16 blocks of a group are packed into one slot of a per-layer pool and given back to the block allocator (all
// but block 0: the first 64 tokens, the sink, stay BF16).
//   pool k_codes / v_codes [slots, hkv, 128, D] uint8 ; k_stats [slots, hkv, D, 2] ; v_stats [slots, hkv, 128, 2]
// ---------------------------------------------------------------------------------------------------------------
// grid (n, hkv), 128 threads; blk_a / blk_b / slot: int32[n] (the two cache blocks of a group and its pool slot).
__global__ void __launch_bounds__(128)
kv_seal_groups_kernel(const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                      const int* __restrict__ blk_a, const int* __restrict__ blk_b, const int* __restrict__ slot,
                      uint8_t* __restrict__ k_codes, uint8_t* __restrict__ v_codes, float* __restrict__ k_stats,
                      float* __restrict__ v_stats, int hkv, int D, int num_blocks, int slots, int* status) {
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ba = blk_a[i], bb = blk_b[i], sl = slot[i];
  if (ba < 0 || ba >= num_blocks || bb < 0 || bb >= num_blocks || sl < 0 || sl >= slots) {
    if (tid == 0) set_status(status, KID_KV, FF_ERR_BOUNDS, i, sl);
    return;
  }
  const size_t obase = ((size_t)sl * hkv + h) * KV_GROUP;           // token row base inside the pool
  // K: thread = channel (D <= 128 per pass)
  for (int d = tid; d < D; d += 128) {
    float lo = 3.402823466e38f, hi = -3.402823466e38f;
    for (int r = 0; r < KV_GROUP; ++r) {
      const int blk = r < 64 ? ba : bb;
      const float x = __bfloat162float(kcache[(((size_t)blk * hkv + h) * 64 + (r & 63)) * D + d]);
      lo = fminf(lo, x); hi = fmaxf(hi, x);
    }
    if (!(fabsf(lo) <= 3.4e38f) || !(fabsf(hi) <= 3.4e38f)) { set_status(status, KID_KV, FF_ERR_NONFINITE, h, sl); lo = 0.f; hi = 0.f; }
    const float span = __fsub_rn(hi, lo), scale = span == 0.f ? 1.f : __fdiv_rn(span, 255.f);
    k_stats[(((size_t)sl * hkv + h) * D + d) * 2] = lo;
    k_stats[(((size_t)sl * hkv + h) * D + d) * 2 + 1] = scale;
    for (int r = 0; r < KV_GROUP; ++r) {
      const int blk = r < 64 ? ba : bb;
      const float x = __bfloat162float(kcache[(((size_t)blk * hkv + h) * 64 + (r & 63)) * D + d]);
      k_codes[(obase + r) * D + d] = kv_code(x, lo, scale);
    }
  }
  // V: one warp per token
  for (int r = warp; r < KV_GROUP; r += 4) {
    const int blk = r < 64 ? ba : bb;
    const __nv_bfloat16* src = vcache + (((size_t)blk * hkv + h) * 64 + (r & 63)) * D;
    float lo = 3.402823466e38f, hi = -3.402823466e38f;
    for (int d = lane; d < D; d += 32) { const float x = __bfloat162float(src[d]); lo = fminf(lo, x); hi = fmaxf(hi, x); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o)); hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o)); }
    if (!(fabsf(lo) <= 3.4e38f) || !(fabsf(hi) <= 3.4e38f)) { if (lane == 0) set_status(status, KID_KV, FF_ERR_NONFINITE, h, sl); lo = 0.f; hi = 0.f; }
    const float span = __fsub_rn(hi, lo), scale = span == 0.f ? 1.f : __fdiv_rn(span, 255.f);
    if (lane == 0) { v_stats[(obase + r) * 2] = lo; v_stats[(obase + r) * 2 + 1] = scale; }
    for (int d = lane; d < D; d += 32) v_codes[(obase + r) * D + d] = kv_code(__bfloat162float(src[d]), lo, scale);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Decode attention over the sealed groups of every sequence (one query row per sequence, head_dim 128): the partial
// (max, sum, weighted values) of each chunk of groups goes into the split-KV partial buffers of the BF16 decode
// kernel, behind its own splits, and the common merge kernel finishes. Keys and values are the dequantised rows
// bf16(code * scale + lo); the soft-max runs in FP32 in the base-2 domain like the BF16 kernel. The first 64
// tokens of group 0 (the sink) are read from BF16 block `block_table[b][0]`.
//   grid (chunks, hkv, batch), 128 threads; group_table [batch, max_groups] pool slots; sealed [batch] tokens sealed
//   part index: ((b * pstride + split_base + chunk) * hq + head)
// ---------------------------------------------------------------------------------------------------------------
constexpr int SEAL_MAXG = 16;      // query heads per KV head (rows of the 16-row MMA tile)
constexpr int SEAL_KEYS = 64;      // keys per soft-max block

// Tensor-core form: the code rows of 64 tokens are de-quantised once into BF16 tiles in shared memory (K with the
// per-channel statistics of the group, V with the per-token ones) and Q Kᵀ and P V run as mma.sync m16n8k16 with the
// G query heads of the KV head as the 16 rows; online soft-max over 64-key blocks in the base-2 domain, P rounded to BF16.
// 128 threads: warp w owns keys 16w .. 16w + 15 of a block in Q Kᵀ and output dims 32w .. 32w + 31 in P V.
__global__ void __launch_bounds__(128)
attn_sealed_kernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ k_codes, const uint8_t* __restrict__ v_codes,
                   const float* __restrict__ k_stats, const float* __restrict__ v_stats,
                   const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                   const int* __restrict__ block_table, const int* __restrict__ group_table, const int* __restrict__ sealed,
                   float* __restrict__ part_o, float* __restrict__ part_ml, int hq, int hkv, int ldq, int max_blocks,
                   int num_blocks, int max_groups, int slots, int groups_per_chunk, int split_base, int pstride,
                   float scale_log2, int* status) {
  pdl_trigger();
  pdl_wait();
  constexpr int D = 128, CH = D / 8;
  __shared__ __align__(128) uint8_t sQ[16 * D * 2];
  __shared__ __align__(128) uint8_t sK[SEAL_KEYS * D * 2];
  __shared__ __align__(128) uint8_t sV[SEAL_KEYS * D * 2];
  __shared__ float sS[16 * SEAL_KEYS];
  __shared__ __align__(16) __nv_bfloat16 sP[16 * SEAL_KEYS];
  __shared__ float sM[16], sL[16], sR[16];
  __shared__ float sk_sc[D], sk_lo[D], sv_sc[SEAL_KEYS], sv_lo[SEAL_KEYS];
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int G = hq / hkv;
  const int ngroups = min(sealed[b] / KV_GROUP, max_groups);
  const int g0 = chunk * groups_per_chunk, g1 = min(ngroups, g0 + groups_per_chunk);
  // Q tile: row r = query head kvh * G + r (rows beyond G are zero)
  for (int i = tid; i < 16 * CH; i += 128) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G) v = *reinterpret_cast<const uint4*>(q + (size_t)b * ldq + (size_t)(kvh * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + ms_off(r, c, CH)) = v;
  }
  if (tid < 16) { sM[tid] = -3.0e38f; sL[tid] = 0.f; }
  float o[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t sQa = smem_u32(sQ), sKa = smem_u32(sK), sVa = smem_u32(sV), sPa = smem_u32(sP);
  __syncthreads();

  for (int grp = g0; grp < g1; ++grp) {
    const int sl = group_table[(size_t)b * max_groups + grp];
    if (sl < 0 || sl >= slots) { if (tid == 0) set_status(status, KID_KV, FF_ERR_BOUNDS, b, grp); break; }
    const size_t tb = ((size_t)sl * hkv + kvh) * KV_GROUP;
    sk_lo[tid] = k_stats[(((size_t)sl * hkv + kvh) * D + tid) * 2];
    sk_sc[tid] = k_stats[(((size_t)sl * hkv + kvh) * D + tid) * 2 + 1];
    for (int half = 0; half < 2; ++half) {
      const bool sink = grp == 0 && half == 0;            // tokens 0..63 of the sequence: BF16 block 0
      __syncthreads();                                    // the previous block's tiles are no longer read; K statistics visible
      if (sink) {
        int blk0 = block_table[(size_t)b * max_blocks];
        if (blk0 < 0 || blk0 >= num_blocks) { if (tid == 0) set_status(status, KID_KV, FF_ERR_BOUNDS, b, blk0); blk0 = 0; }
        const uint4* ks = reinterpret_cast<const uint4*>(kcache + ((size_t)blk0 * hkv + kvh) * 64 * D);
        const uint4* vs = reinterpret_cast<const uint4*>(vcache + ((size_t)blk0 * hkv + kvh) * 64 * D);
        for (int i = tid; i < SEAL_KEYS * CH; i += 128) {
          const int key = i / CH, c = i - key * CH;
          *reinterpret_cast<uint4*>(sK + ms_off(key, c, CH)) = ks[i];
          *reinterpret_cast<uint4*>(sV + ms_off(key, c, CH)) = vs[i];
        }
      } else {
        const size_t row0 = tb + (size_t)half * SEAL_KEYS;
        if (tid < SEAL_KEYS) { sv_lo[tid] = v_stats[(row0 + tid) * 2]; sv_sc[tid] = v_stats[(row0 + tid) * 2 + 1]; }
        // issue all code loads of this thread first (8 x 16 bytes), then convert
        uint4 kc[4], vc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = tid + u * 128;                                   // key = i / 8, 16-code vector = i % 8
          kc[u] = reinterpret_cast<const uint4*>(k_codes + row0 * D)[i];
          vc[u] = reinterpret_cast<const uint4*>(v_codes + row0 * D)[i];
        }
        __syncthreads();                                                  // V statistics visible
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = tid + u * 128, key = i >> 3, v16 = i & 7;
          const uint8_t* kb = reinterpret_cast<const uint8_t*>(&kc[u]);
          const uint8_t* vb = reinterpret_cast<const uint8_t*>(&vc[u]);
          const float vsc = sv_sc[key], vlo = sv_lo[key];
          uint32_t kw[8], vw[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = v16 * 16 + 2 * j;
            kw[j] = pack_bf16x2(fmaf((float)kb[2 * j], sk_sc[c], sk_lo[c]), fmaf((float)kb[2 * j + 1], sk_sc[c + 1], sk_lo[c + 1]));
            vw[j] = pack_bf16x2(fmaf((float)vb[2 * j], vsc, vlo), fmaf((float)vb[2 * j + 1], vsc, vlo));
          }
          *reinterpret_cast<uint4*>(sK + ms_off(key, 2 * v16, CH)) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
          *reinterpret_cast<uint4*>(sK + ms_off(key, 2 * v16 + 1, CH)) = make_uint4(kw[4], kw[5], kw[6], kw[7]);
          *reinterpret_cast<uint4*>(sV + ms_off(key, 2 * v16, CH)) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
          *reinterpret_cast<uint4*>(sV + ms_off(key, 2 * v16 + 1, CH)) = make_uint4(vw[4], vw[5], vw[6], vw[7]);
        }
      }
      __syncthreads();
      // S[16 heads][16 keys of this warp]
      float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4], b0, b1, b2, b3;
        ms_ldsm4(sQa + ms_off((lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4), CH), a[0], a[1], a[2], a[3]);
        ms_ldsm4(sKa + ms_off(warp * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1), CH), b0, b1, b2, b3);
        ms_mma(s[0], a, b0, b1);
        ms_mma(s[1], a, b2, b3);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = warp * 16 + i * 8 + 2 * t + (j & 1), row = g + ((j >> 1) << 3);
          sS[row * SEAL_KEYS + key] = s[i][j] * scale_log2;
        }
      __syncthreads();
      {   // soft-max bookkeeping: 8 threads per head row, 8 keys each
        const int row = tid >> 3, part = tid & 7;
        float sc8[8], mx = -3.0e38f;
#pragma unroll
        for (int j = 0; j < 8; ++j) { sc8[j] = sS[row * SEAL_KEYS + part * 8 + j]; mx = fmaxf(mx, sc8[j]); }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        const float mprev = sM[row], bmax = fmaxf(mprev, mx);
        float bsum = 0.f;
        uint32_t pw[4];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          const float p0 = exp2f(sc8[j] - bmax), p1 = exp2f(sc8[j + 1] - bmax);
          bsum += p0 + p1;
          pw[j >> 1] = pack_bf16x2(p0, p1);
        }
        bsum += __shfl_xor_sync(0xffffffffu, bsum, 1); bsum += __shfl_xor_sync(0xffffffffu, bsum, 2);
        bsum += __shfl_xor_sync(0xffffffffu, bsum, 4);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sP) + ms_off(row, part, 8)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        __syncwarp();
        if (part == 0) {
          const float resc = exp2f(mprev - bmax);
          sR[row] = resc;
          sL[row] = sL[row] * resc + bsum;
          sM[row] = bmax;
        }
      }
      __syncthreads();
      {   // O[16][32 dims of this warp] = O * rescale + P V
        const float r0 = sR[g], r1 = sR[g + 8];
#pragma unroll
        for (int i = 0; i < 4; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
#pragma unroll
        for (int ks = 0; ks < SEAL_KEYS / 16; ++ks) {
          uint32_t pa[4];
          ms_ldsm4(sPa + ms_off((lane & 7) + (((lane >> 3) & 1) << 3), 2 * ks + (lane >> 4), 8), pa[0], pa[1], pa[2], pa[3]);
          const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
          for (int dp = 0; dp < 2; ++dp) {
            uint32_t b0, b1, b2, b3;
            ms_ldsm4t(sVa + ms_off(key, warp * 4 + dp * 2 + (lane >> 4), CH), b0, b1, b2, b3);
            ms_mma(o[2 * dp], pa, b0, b1);
            ms_mma(o[2 * dp + 1], pa, b2, b3);
          }
        }
      }
    }
  }
  __syncthreads();
  // partials of the G heads: (max, sum) and the un-normalised values
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int row = g + 8 * e;
    if (row < G) {
      const size_t pr = ((size_t)b * pstride + split_base + chunk) * hq + (size_t)kvh * G + row;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int d = warp * 32 + i * 8 + 2 * t;
        *reinterpret_cast<float2*>(part_o + pr * D + d) = make_float2(o[i][2 * e], o[i][2 * e + 1]);
      }
      if (warp == 0 && t == 0) { part_ml[pr * 2] = sM[row]; part_ml[pr * 2 + 1] = sL[row]; }
    }
  }
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

// Seal n groups of one layer: blocks (blk_a[i], blk_b[i]) -> pool slot slot[i]. head_dim D (multiple of 32, <= 256).
FF_EXPORT int ff_kv_seal_groups(const void* kcache, const void* vcache, const int* blk_a, const int* blk_b, const int* slot,
                                int n, void* k_codes, void* v_codes, float* k_stats, float* v_stats, int hkv, int D,
                                int num_blocks, int slots, int* status, cudaStream_t s) {
  if (n <= 0 || hkv <= 0 || D <= 0 || D % 32 || D > 256 || num_blocks <= 0 || slots <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(kv_seal_groups_kernel, dim3(n, hkv), dim3(128), 0, s, 0, (const __nv_bfloat16*)kcache,
                          (const __nv_bfloat16*)vcache, blk_a, blk_b, slot, (uint8_t*)k_codes, (uint8_t*)v_codes, k_stats,
                          v_stats, hkv, D, num_blocks, slots, status)) return lr;
  return launch_result();
}

// Partials of the sealed part of a decode step (see attn_sealed_kernel). chunks = ceil(max_groups / groups_per_chunk)
// splits are written for every (sequence, head), neutral where a sequence has nothing sealed there.
FF_EXPORT int ff_attn_sealed(const void* q, const void* k_codes, const void* v_codes, const float* k_stats,
                             const float* v_stats, const void* kcache, const void* vcache, const int* block_table,
                             const int* group_table, const int* sealed, float* part_o, float* part_ml, int batch, int hq,
                             int hkv, int head_dim, int ldq, int max_blocks, int num_blocks, int max_groups, int slots,
                             int groups_per_chunk, int split_base, int pstride, float scale, int* status, cudaStream_t s) {
  if (batch <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || hq / hkv > SEAL_MAXG || head_dim != 128) return FF_HOST_BAD_SHAPE;
  if (max_groups <= 0 || groups_per_chunk <= 0 || slots <= 0 || !(scale > 0.f)) return FF_HOST_BAD_SHAPE;
  const int chunks = (max_groups + groups_per_chunk - 1) / groups_per_chunk;
  if (split_base < 0 || split_base + chunks > pstride) return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(k_codes) & 15) || (reinterpret_cast<uintptr_t>(kcache) & 15)) return FF_HOST_BAD_ALIGN;
  if (int lr = launch_pdl(attn_sealed_kernel, dim3(chunks, hkv, batch), dim3(128), 0, s, 0, (const __nv_bfloat16*)q,
                          (const uint8_t*)k_codes, (const uint8_t*)v_codes, k_stats, v_stats, (const __nv_bfloat16*)kcache,
                          (const __nv_bfloat16*)vcache, block_table, group_table, sealed, part_o, part_ml, hq, hkv, ldq,
                          max_blocks, num_blocks, max_groups, slots, groups_per_chunk, split_base, pstride,
                          scale * 1.4426950408889634f, status)) return lr;
  return launch_result();
}
