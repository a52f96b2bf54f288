// Multi-head latent attention (DeepSeek-style MLA) over a paged latent cache, absorbed form.
//
// The cache stores ONE row per token: [ c_kv (kv_lora_rank = 512) | k_rope (64) ] = 576 BF16 values
// (block layout [block][1][64][576]); every query head attends to it as multi-query attention:
//     score = q_lat · c_kv + q_rope · k_rope ,  out_lat = softmax(score) · c_kv
// where q_lat = q_nope · W_UK was absorbed by the caller and out_lat is projected by W_UV afterwards.
// One CTA owns 16 packed (query position, head) rows of one sequence; its four warps all compute the
// 16 x 64 score tile of a page (Q tile in shared memory, 576-wide dot products on mma.sync) and each
// accumulates a 128-wide slice of the 512-wide output, so the softmax state needs no cross-warp
// merge. Pages stream through a cp.async double buffer; optional split-KV for decode.
// The reference serves DeepSeek with a latent window / indexed attention family
// (kernels/latent_window_attention.cu, latent_indexed_attention); this kernel is the paged
// full-context member of that family.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {
namespace mla {

constexpr int LD = 576;            // latent + rope dims of a cache row
constexpr int LV = 512;            // value dims (the latent part)
constexpr int PAGE = 64;
constexpr int CH = LD / 8;         // 16-byte chunks per row = 72
constexpr float NEG_BIG = -3.0e38f;

__device__ __forceinline__ void cp_async16(void* s, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(s)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm4t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of chunk c of row r: XOR the low three chunk bits with the row
__device__ __forceinline__ uint32_t toff(int r, int c) { return (uint32_t)((r * CH + ((c & ~7) | ((c ^ r) & 7))) * 16); }

// q       : [total rows][heads][576] bf16 (row = query position, packed per sequence via q_start)
// out     : [total rows][heads][512] bf16
// part_o  : fp32 [B][nsplit][max_rows][512], part_ml fp32 [B][nsplit][max_rows][2]  (max_rows = max_q * heads)
// grid (pairs of 16-row tiles, nsplit, B), 256 threads
__global__ void __launch_bounds__(256)
mla_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                const int* __restrict__ block_table, const int* __restrict__ q_start, const int* __restrict__ q_lens,
                const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                float* __restrict__ part_ml, int heads, int max_blocks, int num_blocks, int nsplit, int max_rows,
                float scale_log2, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  // two 16-row tiles per CTA (warps 0-3 and 4-7) share the K pages in shared memory: half the page traffic and twice
  // the warps per SM of a one-tile CTA
  const int split = blockIdx.y, b = blockIdx.z;
  const int qlen = q_lens[b], ctx = ctx_lens[b], qs = q_start[b];
  const int rows_total = qlen * heads;
  if (blockIdx.x * 32 >= rows_total) return;
  const int tile = threadIdx.x >> 7;                    // 0 / 1
  const int rt = blockIdx.x * 2 + tile;
  const int tid = threadIdx.x & 127;                    // thread within the tile's four warps
  const int warp = tid >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  uint8_t* sQ = smem + tile * 18432;                    // 16 x 576 bf16 = 18432 B per tile
  uint8_t* sK[2] = {smem + 2 * 18432, smem + 2 * 18432 + PAGE * LD * 2};
  const int past = ctx - qlen;

  // Q tile -> shared memory (zero rows beyond the sequence's rows)
  for (int i = tid; i < 16 * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const int rg = rt * 16 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rg < rows_total) v = *reinterpret_cast<const uint4*>(q + ((size_t)(qs + rg / heads) * heads + rg % heads) * LD + c * 8);
    *reinterpret_cast<uint4*>(sQ + toff(r, c)) = v;
  }
  int lim[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int rg = rt * 16 + g + e * 8;
    lim[e] = rg < rows_total ? past + rg / heads : -1;
  }
  const int last_row = min(rows_total, blockIdx.x * 32 + 32) - 1;     // both tiles walk the same pages
  const int last_key = past + last_row / heads;
  const int pages = last_key / PAGE + 1;
  const int per = (pages + nsplit - 1) / nsplit;
  const int p0 = split * per, p1 = min(pages, p0 + per);

  // score tile, probabilities and the soft-max state of the 16 rows live in shared memory: every warp computes the
  // scores of its own 16 keys of a page (no redundant Q K^T), the rows' state is updated once, and every warp then
  // accumulates its 128-wide slice of P V
  constexpr int TILE_AUX = 16 * PAGE * 4 + 16 * PAGE * 2 + 3 * 16 * 4;
  uint8_t* aux = smem + 2 * 18432 + 2 * PAGE * LD * 2 + tile * TILE_AUX;
  float* sS = reinterpret_cast<float*>(aux);                                       // [16][64] f32
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sS + 16 * PAGE);            // [16][64] bf16, chunk-swizzled
  float* sM = reinterpret_cast<float*>(sP + 16 * PAGE);                            // [16] running max
  float* sL = sM + 16;                                                             // [16] running sum
  float* sR = sL + 16;                                                             // [16] rescale of this page
  if (tid < 16) { sM[tid] = NEG_BIG; sL[tid] = 0.f; }
  float o[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  bool bad = false;
  auto issue = [&](int page, int buf) {
    int blk = block_table[(size_t)b * max_blocks + page];
    if (blk < 0 || blk >= num_blocks) { bad = true; blk = 0; }
    const __nv_bfloat16* src = cache + (size_t)blk * PAGE * LD;
    for (int i = threadIdx.x; i < PAGE * CH; i += 256) {
      const int r = i / CH, c = i % CH;
      cp_async16(sK[buf] + toff(r, c), src + (size_t)r * LD + c * 8);
    }
    cp_commit();
  };
  if (p0 < p1) issue(p0, 0);
  const uint32_t sQa = smem_u32(sQ), sPa = smem_u32(sP);
  for (int p = p0; p < p1; ++p) {
    const int buf = (p - p0) & 1;
    if (p + 1 < p1) { issue(p + 1, buf ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
    __syncthreads();
    const uint32_t sKa = smem_u32(sK[buf]);
    // S[16 rows][16 keys of this warp]
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll 4
    for (int kk = 0; kk < LD / 16; ++kk) {
      uint32_t a[4], b0, b1, b2, b3;
      ldsm4(sQa + toff((lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4)), a[0], a[1], a[2], a[3]);
      ldsm4(sKa + toff(warp * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1)), b0, b1, b2, b3);
      mma(s[0], a, b0, b1);
      mma(s[1], a, b2, b3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kcol = warp * 16 + i * 8 + 2 * t + (j & 1), row = g + ((j >> 1) << 3);
        const bool vis = p * PAGE + kcol <= ((j < 2) ? lim[0] : lim[1]);
        sS[row * PAGE + kcol] = vis ? s[i][j] * scale_log2 : NEG_BIG;
      }
    __syncthreads();
    {   // soft-max bookkeeping: 8 threads per row, 8 keys each
      const int row = tid >> 3, part = tid & 7;
      float sc8[8], mx = NEG_BIG;
#pragma unroll
      for (int j = 0; j < 8; ++j) { sc8[j] = sS[row * PAGE + part * 8 + j]; mx = fmaxf(mx, sc8[j]); }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mprev = sM[row], bmax = fmaxf(mprev, mx);
      float bsum = 0.f;
      uint32_t pw[4];
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float p0v = (sc8[j] <= NEG_BIG) ? 0.f : exp2f(sc8[j] - bmax);
        const float p1v = (sc8[j + 1] <= NEG_BIG) ? 0.f : exp2f(sc8[j + 1] - bmax);
        bsum += p0v + p1v;
        pw[j >> 1] = pack_bf16x2(p0v, p1v);
      }
      bsum += __shfl_xor_sync(0xffffffffu, bsum, 1); bsum += __shfl_xor_sync(0xffffffffu, bsum, 2);
      bsum += __shfl_xor_sync(0xffffffffu, bsum, 4);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sP) + ((row * 8 + (part ^ (row & 7))) * 16)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      __syncwarp();
      if (part == 0) {
        const float resc = exp2f(mprev - bmax);
        sR[row] = resc;
        sL[row] = sL[row] * resc + bsum;
        sM[row] = bmax;
      }
    }
    __syncthreads();
    {   // O[16][128 dims of this warp] = O * rescale + P V
      const float r0s = sR[g], r1s = sR[g + 8];
#pragma unroll
      for (int i = 0; i < 16; ++i) { o[i][0] *= r0s; o[i][1] *= r0s; o[i][2] *= r1s; o[i][3] *= r1s; }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t pa[4];
        {
          const int prow = (lane & 7) + (((lane >> 3) & 1) << 3), pch = 2 * ks + (lane >> 4);
          ldsm4(sPa + (uint32_t)((prow * 8 + (pch ^ (prow & 7))) * 16), pa[0], pa[1], pa[2], pa[3]);
        }
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          uint32_t b0, b1, b2, b3;
          ldsm4t(sKa + toff(key, warp * 16 + dp * 2 + (lane >> 4)), b0, b1, b2, b3);
          mma(o[2 * dp], pa, b0, b1);
          mma(o[2 * dp + 1], pa, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  if (bad) set_status(status, KID_MLA, FF_ERR_BOUNDS, b, rt);
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int rg = rt * 16 + g + e * 8;
    if (rg >= rows_total) continue;
    const float L = sL[g + 8 * e];
    if (nsplit == 1) {
      const float inv = L > 0.f ? 1.f / L : 0.f;
      __nv_bfloat16* dst = out + ((size_t)(qs + rg / heads) * heads + rg % heads) * LV + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i)
        *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t) = pack_bf16x2(o[i][2 * e] * inv, o[i][2 * e + 1] * inv);
    } else {
      const size_t pr = ((size_t)b * nsplit + split) * max_rows + rg;
      float* dst = part_o + pr * LV + warp * 128;
#pragma unroll
      for (int i = 0; i < 16; ++i) { dst[i * 8 + 2 * t] = o[i][2 * e]; dst[i * 8 + 2 * t + 1] = o[i][2 * e + 1]; }
      if (warp == 0 && t == 0) { part_ml[pr * 2] = sM[g + 8 * e]; part_ml[pr * 2 + 1] = L; }
    }
  }
}

// grid (max_rows, B), 128 threads x 4 dims
__global__ void __launch_bounds__(128)
mla_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                 const int* __restrict__ q_start, const int* __restrict__ q_lens, int heads, int nsplit, int max_rows) {
  const int rg = blockIdx.x, b = blockIdx.y;
  if (rg >= q_lens[b] * heads) return;
  float M = NEG_BIG;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(((size_t)b * nsplit + s) * max_rows + rg) * 2]);
  float L = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < nsplit; ++s) {
    const size_t pr = ((size_t)b * nsplit + s) * max_rows + rg;
    const float sc = exp2f(part_ml[pr * 2] - M);
    L += part_ml[pr * 2 + 1] * sc;
    const float4 v = *reinterpret_cast<const float4*>(part_o + pr * LV + threadIdx.x * 4);
    acc[0] += v.x * sc; acc[1] += v.y * sc; acc[2] += v.z * sc; acc[3] += v.w * sc;
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  __nv_bfloat16* dst = out + ((size_t)(q_start[b] + rg / heads) * heads + rg % heads) * LV + threadIdx.x * 4;
  *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(acc[0] * inv, acc[1] * inv), pack_bf16x2(acc[2] * inv, acc[3] * inv));
}

// latent cache write: row r -> cache[slot] = [c (512) | k_rope (64)]; slot < 0 skips
__global__ void mla_cache_write_kernel(const __nv_bfloat16* __restrict__ c, const __nv_bfloat16* __restrict__ kr,
                                       const int* __restrict__ slots, __nv_bfloat16* __restrict__ cache, int rows,
                                       int ldc, int ldk, int num_blocks, int* status) {
  const int row = blockIdx.x;
  const int slot = slots[row];
  if (slot < 0) return;
  if (slot >= num_blocks * PAGE) { set_status(status, KID_MLA, FF_ERR_BOUNDS, row, slot); return; }
  __nv_bfloat16* dst = cache + (size_t)slot * LD;
  for (int v = threadIdx.x; v < CH; v += blockDim.x) {
    const uint4 x = v < LV / 8 ? reinterpret_cast<const uint4*>(c + (size_t)row * ldc)[v]
                               : reinterpret_cast<const uint4*>(kr + (size_t)row * ldk)[v - LV / 8];
    reinterpret_cast<uint4*>(dst)[v] = x;
  }
}

}  // namespace mla
}  // namespace ff
using namespace ff;

constexpr int MLA_SMEM = 2 * 18432 + 2 * mla::PAGE * mla::LD * 2 + 2 * (16 * mla::PAGE * 4 + 16 * mla::PAGE * 2 + 3 * 16 * 4);   // two Q tiles + two page stages + per-tile score / probability tiles and row state

FF_EXPORT int ff_mla_plan(int batch, int heads, int max_q, int max_ctx, long long* part_o_bytes, long long* part_ml_bytes) {
  const int tiles = (max_q * heads + 31) / 32;        // a CTA owns two 16-row tiles
  const int ctas = batch * tiles;
  int nsplit = 1;
  if (ctas < 148) nsplit = (148 + ctas - 1) / ctas;
  const int pages = (max_ctx + mla::PAGE - 1) / mla::PAGE;
  if (nsplit > pages) nsplit = pages;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 32) nsplit = 32;
  if (part_o_bytes) *part_o_bytes = (long long)batch * nsplit * max_q * heads * mla::LV * 4;
  if (part_ml_bytes) *part_ml_bytes = (long long)batch * nsplit * max_q * heads * 2 * 4;
  return nsplit;
}

FF_EXPORT int ff_mla_attn(const void* q, const void* cache, const int* block_table, const int* q_start, const int* q_lens,
                          const int* ctx_lens, void* out, float* part_o, float* part_ml, int batch, int heads, int max_q,
                          int max_blocks, int num_blocks, int nsplit, float scale, int* status, cudaStream_t s) {
  if (batch <= 0 || heads <= 0 || max_q <= 0 || nsplit < 1) return FF_HOST_BAD_SHAPE;
  if (nsplit > 1 && (!part_o || !part_ml)) return FF_HOST_BAD_SHAPE;
  if (int r = opt_in_smem(mla::mla_attn_kernel, MLA_SMEM)) return r;
  const int max_rows = max_q * heads;
  dim3 grid((max_rows + 31) / 32, nsplit, batch);
  mla::mla_attn_kernel<<<grid, 256, MLA_SMEM, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)cache, block_table,
      q_start, q_lens, ctx_lens, (__nv_bfloat16*)out, part_o, part_ml, heads, max_blocks, num_blocks, nsplit, max_rows,
      scale * 1.4426950408889634f, status);
  if (int r = launch_result()) return r;
  if (nsplit > 1) {
    dim3 g2(max_rows, batch);
    mla::mla_merge_kernel<<<g2, 128, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, q_start, q_lens, heads, nsplit, max_rows);
    return launch_result();
  }
  return 0;
}

FF_EXPORT int ff_mla_cache_write(const void* c, const void* k_rope, const int* slots, void* cache, int rows, int ldc,
                                 int ldk, int num_blocks, int* status, cudaStream_t s) {
  if (rows <= 0 || ldc % 8 || ldk % 8) return FF_HOST_BAD_SHAPE;
  mla::mla_cache_write_kernel<<<rows, 96, 0, s>>>((const __nv_bfloat16*)c, (const __nv_bfloat16*)k_rope, slots,
                                                  (__nv_bfloat16*)cache, rows, ldc, ldk, num_blocks, status);
  return launch_result();
}
