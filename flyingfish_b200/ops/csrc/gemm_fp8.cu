// Block-scaled FP8 (E4M3) linear on tcgen05:  Y[M,N] = dequant(Xq)[M,K] · dequant(Wq)[N,K]ᵀ
//   Wq : E4M3 codes [N,K] with one FP32 scale per 128x128 block (DeepSeek-V3 checkpoint layout)
//   Xq : E4M3 codes [M,K] with one FP32 scale per 1x128 (activation quantised by quantize.cu)
// The tensor core multiplies the raw codes (kind::f8f6f4, FP32 accumulation in TMEM) one 128-wide
// K block at a time; the epilogue warps pull each block's partial sums out of TMEM and add them
// into FP32 registers multiplied by w_scale[block] * x_scale[token, block] -- the same "per-K-block
// partial times (w_scale * x_scale)" contract as the reference's fp8_block kernels
// (kernels/fp8_linear.cu:73-140), which run on mma.sync and fall back to a BF16 materialisation +
// cuBLAS for large M. Two (four for at most 64 tokens) TMEM accumulators let later blocks multiply while block k is promoted.
//
// Swap-AB like the BF16 decode kernel: a 128-row weight tile (exactly one scale-block row) is
// the UMMA A operand, up to 128 tokens are the UMMA N dimension. Dense use: grid (N/128, splits),
// split-K partials go through FP32 scratch and the last CTA of a tile adds them in split order.
// 320 threads: one TMA warp, one MMA warp, eight promoting warps.
// Grouped (MoE) use: grid (Nw/128, 1, experts) over 16-row padded expert segments, optional
// SwiGLU epilogue for gate/up weights interleaved per 64 rows.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int FBM = 128, FBK = 128, F_TOK = 128, F_STAGES_MAX = 12;

struct alignas(8) Fp8Bars {
  uint64_t full[F_STAGES_MAX];
  uint64_t empty[F_STAGES_MAX];
  uint64_t tmem_full[4];
  uint64_t tmem_empty[4];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ float silu_f8(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float bfr8(float x) { return __bfloat162float(__float2bfloat16(x)); }

// Promotion of P consecutive k-blocks for a warp that owns `nb` (<= U) 16-column blocks: all tensor-memory loads are
// issued before the single wait, so the fixed latency of the wait -> load -> arrive chain is paid once per call.
// acc[16 u + j] += partial[u][j] * scale[u][j], k-blocks in order (the summation order of the contract).
template <int U, int P, int OFF, int NACC>
__device__ __forceinline__ void fp8_promote(float (&acc)[NACC], const uint32_t (&taddr)[2], const float* const (&sp)[2],
                                            int nb) {
  uint32_t r[P][U][16];
#pragma unroll
  for (int p = 0; p < P; ++p)
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (OFF / 16 + u < nb) tmem_ld_x16(taddr[p] + OFF + 16 * u, r[p][u]);
  tmem_ld_wait();
#pragma unroll
  for (int p = 0; p < P; ++p)
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (OFF / 16 + u < nb) {
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 sc = *reinterpret_cast<const float4*>(sp[p] + OFF + 16 * u + 4 * j4);
          acc[OFF + 16 * u + 4 * j4 + 0] += __uint_as_float(r[p][u][4 * j4 + 0]) * sc.x;
          acc[OFF + 16 * u + 4 * j4 + 1] += __uint_as_float(r[p][u][4 * j4 + 1]) * sc.y;
          acc[OFF + 16 * u + 4 * j4 + 2] += __uint_as_float(r[p][u][4 * j4 + 2]) * sc.z;
          acc[OFF + 16 * u + 4 * j4 + 3] += __uint_as_float(r[p][u][4 * j4 + 3]) * sc.w;
        }
      }
    }
}

// epi: 0 store, 1 SwiGLU over 64/64 interleaved rows (grouped gate/up)
// TOK: tokens per chunk. 128 for prefill-sized and dense calls (one CTA per SM); 32 for decode-sized grouped calls, where a
// CTA needs few registers and half the shared memory so that two CTAs share an SM and one streams while the other sets up
// or drains (an expert tile of a decode batch is short: 16 to 56 k-blocks).
template <int TOK>
__global__ void __launch_bounds__(320, TOK <= 32 ? 2 : 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const float* __restrict__ w_scale, const float* __restrict__ x_scale, __nv_bfloat16* __restrict__ Y,
                const int* __restrict__ seg_off, const int* __restrict__ counts, int M, int Nw, int K, int ldy,
                int epi, int splits, int pipe_bytes, int stage_off, int tok_cap, float* __restrict__ scratch,
                int* __restrict__ tile_counters, int* status, int xs_ld) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Fp8Bars bars;
  const int tn = blockIdx.x, split = blockIdx.y, e = blockIdx.z;
  const int row0 = seg_off ? seg_off[e] : 0;
  // a segment that reaches past the row buffers (a dispatch that overflowed its capacity and said so through the status
  // word) is cut at the buffer end: no row beyond M is read or written
  const int cnt = counts ? min(counts[e], M - row0) : M;
  if (cnt <= 0) return;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // staging is sized by the host for the tokens of this launch (tok_cap) and the k-blocks of one split: what it
  // does not take is pipeline depth, and the bytes in flight per SM are what bounds the weight stream
  __nv_bfloat16* sT = reinterpret_cast<__nv_bfloat16*>(smem);            // [tok_cap][128] bf16
  float* sXs = reinterpret_cast<float*>(smem + tok_cap * FBM * 2);       // scale products [ntok][nkb]
  uint8_t* pipe = smem + stage_off;
  constexpr int A_BYTES = FBM * FBK;                                     // 16 KiB of E4M3
  const int kblocks_total = (K + FBK - 1) / FBK;
  const int per = (kblocks_total + splits - 1) / splits;
  const int kb0 = split * per, kb1 = min(kblocks_total, kb0 + per);
  const int nkb = max(0, kb1 - kb0);
  const int ntok_max = min(TOK, ((cnt + 15) / 16) * 16);
  const int stage_bytes = A_BYTES + ntok_max * FBK;
  const int stages = min(F_STAGES_MAX, pipe_bytes / stage_bytes);
  const int chunks = (cnt + TOK - 1) / TOK;
  // accumulators in tensor memory: four of 64 columns when the launch has at most 64 tokens per chunk, else two of 128.
  // The multiplies of up to three k-blocks run ahead of the promotion of the first, which hides the commit -> wait ->
  // load -> arrive latency chain between the MMA thread and the promoting warps.
  const int nbuf = ntok_max <= 64 ? 4 : 2;
  const int buf_cols = 256 / nbuf;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int scale_rows = (Nw + 127) / 128;                                // scale rows per expert

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 4; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 8); }
    bars.abort_flag = 0; bars.is_last = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  pdl_trigger();
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX);
      uint32_t it = 0; bool ok = true;
      // the weights do not depend on the kernel before this one (which produced the activation codes and scales):
      // the weight tiles of the first stages are requested before the dependency wait, the activation tiles after it
      const int ntok0 = min(TOK, ((cnt + 15) / 16) * 16);
      const int pre = min(stages, nkb);
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&bars.full[i], A_BYTES + ntok0 * FBK);
        tma_load_2d(pipe + i * stage_bytes, &tmW, &bars.full[i], (kb0 + i) * FBK, e * Nw + tn * FBM);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        for (int r = 0; r < ntok0; r += 16)
          tma_load_2d(pipe + i * stage_bytes + A_BYTES + r * FBK, &tmX, &bars.full[i], (kb0 + i) * FBK, row0 + r);
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(TOK, ((cnt - c * TOK + 15) / 16) * 16);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if (c == 0 && kb - kb0 < pre) continue;                 // requested above
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_FP8, 1)) { ok = false; break; }
          if (blockIdx.x == 0 && blockIdx.y == 0) FF_TL(status, KID_GEMM_FP8, 10);
          mbar_expect_tx(&bars.full[s], A_BYTES + ntok * FBK);
          uint8_t* sa = pipe + s * stage_bytes;
          tma_load_2d(sa, &tmW, &bars.full[s], kb * FBK, e * Nw + tn * FBM);
          for (int r = 0; r < ntok; r += 16)
            tma_load_2d(sa + A_BYTES + r * FBK, &tmX, &bars.full[s], kb * FBK, row0 + c * TOK + r);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, kit = 0; bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(TOK, ((cnt - c * TOK + 15) / 16) * 16);
        const uint32_t idesc = umma_idesc(0, 0, 0, 0, FBM, ntok);        // E4M3 x E4M3 -> FP32
        for (int kb = kb0; kb < kb1; ++kb, ++it, ++kit) {
          const int b = kit % nbuf; const uint32_t bph = (kit / nbuf) & 1;
          if (!mbar_wait(&bars.tmem_empty[b], bph ^ 1, abort_flag, status, KID_GEMM_FP8, 2)) { ok = false; break; }
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (blockIdx.x == 0 && blockIdx.y == 0) FF_TL(status, KID_GEMM_FP8, 20);
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_GEMM_FP8, 3)) { ok = false; break; }
          if (blockIdx.x == 0 && blockIdx.y == 0) FF_TL(status, KID_GEMM_FP8, 21);
          tc_fence_after();
          const uint32_t sa = smem_u32(pipe + s * stage_bytes);
          const uint64_t da = umma_desc_sw128(sa, 16, 1024);
          const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < FBK / 32; ++k) umma_f8f6f4(tmem_base + b * buf_cols, da + 2 * k, db + 2 * k, idesc, k != 0);
          umma_commit(&bars.empty[s]);
          umma_commit(&bars.tmem_full[b]);
        }
      }
    }
  } else {
    // eight promoting warps: two per 32-lane quadrant of tensor memory, each owning half of the token columns
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int nl = q * 32 + lane;
    const int ee = (warp - 2) * 32 + lane;                 // 0 .. 255
    const int n = tn * FBM + nl;
    const float* ws_row = w_scale + ((size_t)e * scale_rows + tn) * kblocks_total;
    uint32_t kit = 0; bool ok = true;
    pdl_wait();                                   // activation scales, scratch, counters and Y belong to earlier kernels until here
    for (int c = 0; c < chunks && ok; ++c) {
      const int ntok = min(TOK, ((cnt - c * TOK + 15) / 16) * 16);
      const int real = min(TOK, cnt - c * TOK);
      const int grow0 = row0 + c * TOK;
      const int nblk = ntok / 16;                           // 16-column blocks of this chunk
      const int blk0 = half == 0 ? 0 : (nblk + 1) / 2;      // this warp's blocks: [blk0, blk1)
      const int blk1 = half == 0 ? (nblk + 1) / 2 : nblk;
      // scale products of this chunk and K range -> shared memory [kb][ntok] (the product of the two scales is what
      // every partial sum is multiplied by: staged once, so that no global load sits between a k-block's arrival and
      // its promotion); eight independent loads per thread in flight
      for (int i0 = ee; i0 < ntok * nkb; i0 += 256 * 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * 256;
          v[u] = 0.f;
          if (i < ntok * nkb) {
            const int t = i / nkb, kb = i - t * nkb;
            if (t < real) v[u] = ws_row[kb0 + kb] * x_scale[(size_t)(grow0 + t) * xs_ld + kb0 + kb];
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * 256;
          if (i < ntok * nkb) { const int t = i / nkb, kb = i - t * nkb; sXs[kb * ntok + t] = v[u]; }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      float acc[TOK / 2];                                 // columns (blk0 + i / 16) * 16 + i % 16
#pragma unroll
      for (int i = 0; i < TOK / 2; ++i) acc[i] = 0.f;
      const int nb = blk1 - blk0;
      for (int kb = 0; kb < nkb && ok; ++kb, ++kit) {
        const int b0 = kit % nbuf;
        if (!mbar_wait(&bars.tmem_full[b0], (kit / nbuf) & 1, abort_flag, status, KID_GEMM_FP8, 4)) { ok = false; break; }
        if (blockIdx.x == 0 && blockIdx.y == 0 && ee == 0) FF_TL(status, KID_GEMM_FP8, 30);
        tc_fence_after();
        const uint32_t lane_base = tmem_base + (uint32_t(q * 32) << 16) + blk0 * 16;
        const uint32_t taddr[2] = {lane_base + b0 * buf_cols, 0};
        const float* const sp[2] = {sXs + kb * ntok + blk0 * 16, nullptr};
        // (promoting two k-blocks per round was measured: the extra registers spill under the 168-register cap of a
        // ten-warp CTA and the kernel gets slower)
        fp8_promote<TOK / 32, 1, 0, TOK / 2>(acc, taddr, sp, nb);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tmem_empty[b0]);
        if (blockIdx.x == 0 && blockIdx.y == 0 && ee == 0) FF_TL(status, KID_GEMM_FP8, 31);
      }
      if (!ok) break;
      bool final_here = true;
      if (splits == 1) {
#pragma unroll
        for (int i = 0; i < TOK / 2; ++i) {
          const int t = blk0 * 16 + i;
          if (t < blk1 * 16) sT[t * FBM + nl] = __float2bfloat16(acc[i]);
        }
      } else {
        float* part = scratch + ((size_t)split * M) * Nw;
#pragma unroll
        for (int i = 0; i < TOK / 2; ++i) {
          const int t = blk0 * 16 + i;
          if (t < blk1 * 16 && t < real && n < Nw) part[(size_t)(grow0 + t) * Nw + n] = acc[i];
        }
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ee == 0) {
          const int prev = atomicAdd(&tile_counters[tn * chunks + c], 1);
          bars.is_last = (prev == splits - 1);
          if (prev == splits - 1) tile_counters[tn * chunks + c] = 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        final_here = bars.is_last != 0;
        if (final_here) {
          __threadfence();
          // partials are added in split order (fixed summation order). Thread -> four adjacent columns and every
          // eighth token: eight 16-byte loads of one split in flight per thread, the sums go straight into the staging tile
          const int c4 = (ee & 31) * 4, tg = ee >> 5;          // tg 0 .. 7
          const int ncol = tn * FBM + c4;
          const bool vec = (Nw & 3) == 0 && ncol + 3 < Nw;
          for (int tb = 0; tb < ntok; tb += 64) {              // bands of 64 tokens: eight tokens per thread and band
            float4 sum[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < splits; ++s) {
              const float* ps = scratch + ((size_t)s * M + grow0) * Nw + ncol;
              float4 v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int t = tb + tg + 8 * j;
                v[j] = (t < real && vec) ? __ldcg(reinterpret_cast<const float4*>(ps + (size_t)t * Nw))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < real && !vec) {                        // ragged right edge, or rows that are not 16-byte aligned
                  float e4[4] = {0.f, 0.f, 0.f, 0.f};
                  for (int q2 = 0; q2 < 4 && ncol + q2 < Nw; ++q2) e4[q2] = __ldcg(ps + (size_t)t * Nw + q2);
                  v[j] = make_float4(e4[0], e4[1], e4[2], e4[3]);
                }
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) { sum[j].x += v[j].x; sum[j].y += v[j].y; sum[j].z += v[j].z; sum[j].w += v[j].w; }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int t = tb + tg + 8 * j;
              if (t < ntok) {
                __nv_bfloat162* d = reinterpret_cast<__nv_bfloat162*>(sT + t * FBM + c4);
                d[0] = __floats2bfloat162_rn(sum[j].x, sum[j].y);
                d[1] = __floats2bfloat162_rn(sum[j].z, sum[j].w);
              }
            }
          }
        }
      }
      if (final_here) {
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (epi == 1) {
          const int c8 = ee & 7, r0 = ee >> 3;
          for (int t = r0; t < real; t += 32) {
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = c8 * 8 + 2 * j;
              const float g0 = __bfloat162float(sT[t * FBM + col]), g1 = __bfloat162float(sT[t * FBM + col + 1]);
              const float u0 = __bfloat162float(sT[t * FBM + 64 + col]), u1 = __bfloat162float(sT[t * FBM + 64 + col + 1]);
              o[j] = pack_bf16x2(bfr8(silu_f8(g0)) * u0, bfr8(silu_f8(g1)) * u1);
            }
            *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t) * ldy + tn * 64 + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          const int c16 = ee & 15, r0 = ee >> 4;
          const int col = tn * FBM + c16 * 8;
          if (col + 8 <= Nw) {
            for (int t = r0; t < real; t += 16)
              *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t) * ldy + col) = *reinterpret_cast<const uint4*>(sT + t * FBM + c16 * 8);
          } else if (col < Nw) {
            for (int t = r0; t < real; t += 16)
              for (int j = 0; j < 8 && col + j < Nw; ++j) Y[(size_t)(grow0 + t) * ldy + col + j] = sT[t * FBM + c16 * 8 + j];
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
  }
  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_gemm_fp8_plan(int M, int N, int K, long long* scratch_bytes, long long* counter_bytes) {
  const int tiles = (N + FBM - 1) / FBM;
  const int kblocks = (K + FBK - 1) / FBK;
  const int chunks = (M + F_TOK - 1) / F_TOK;      // dense calls always use 128-token chunks
  int splits = 1;
  if (tiles * chunks < 148) {
    splits = 148 / (tiles * chunks);
    const int maxs = kblocks / 4 > 0 ? kblocks / 4 : 1;
    if (splits > maxs) splits = maxs;
    if (splits < 1) splits = 1;
  }
  if (scratch_bytes) *scratch_bytes = splits > 1 ? (long long)splits * M * N * 4 : 0;
  if (counter_bytes) *counter_bytes = (long long)tiles * chunks * 4;
  return splits;
}

// Dense: seg_off = counts = null, experts = 1. Grouped: W is [experts*Nw, K], w_scale
// [experts*ceil(Nw/128), K/128], X / x_scale are the 16-row padded sorted buffers, M = capacity.
static int gemm_fp8_launch(const void* xq, const float* x_scale, const void* wq, const float* w_scale, void* y,
                           const int* seg_off, const int* counts, int experts, int M, int Nw, int K, int ldy, int epi,
                           int splits, float* scratch, int* tile_counters, int* status, cudaStream_t s, long long ldxq,
                           int xs_ld) {
  if (ldxq < K || ldxq % 16 || xs_ld < K / 128) return FF_HOST_BAD_SHAPE;
  if (M <= 0 || Nw <= 0 || K <= 0 || K % 128 || experts < 1) return FF_HOST_BAD_SHAPE;
  if (experts > 1 && (!seg_off || !counts || Nw % 128)) return FF_HOST_BAD_SHAPE;
  if (splits < 1 || (splits > 1 && (!scratch || !tile_counters || experts > 1))) return FF_HOST_BAD_SHAPE;
  if (epi == 1 && (Nw % 128 || ldy < Nw / 2)) return FF_HOST_BAD_SHAPE;
  if (ldy % 8 || (reinterpret_cast<uintptr_t>(y) & 15)) return FF_HOST_BAD_ALIGN;
  // decode-sized grouped calls (on average at most 24 padded rows per expert): 32-token chunks, two CTAs per SM
  const bool small = experts > 1 ? (long long)M <= 24ll * experts : M <= 32;
  const int tok_cap = small ? (experts > 1 ? 32 : (M + 15) / 16 * 16) : (experts > 1 ? F_TOK : (M >= F_TOK ? F_TOK : (M + 15) / 16 * 16));
  const int per = ((K / 128) + splits - 1) / splits;                     // k-blocks of one split
  if (per * tok_cap * 4 > 64 * 1024) return FF_HOST_TOO_LARGE;           // scale staging
  CUtensorMap tmW, tmX;
  int r = make_tmap_2d(&tmW, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, (uint64_t)experts * Nw, (uint64_t)K, FBK, FBM);
  if (r) return r;
  r = make_tmap_2d(&tmX, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, (uint64_t)ldxq, FBK, 16);
  if (r) return r;
  const int staging = (tok_cap * FBM * 2 + per * tok_cap * 4 + 1023) / 1024 * 1024;
  const int budget = small ? 110 * 1024 : 224 * 1024;
  int pipe_bytes = budget - staging;
  const int smem = staging + pipe_bytes + 1024;
  dim3 grid((Nw + FBM - 1) / FBM, splits, experts);
  if (small) {
    r = opt_in_smem(gemm_fp8_kernel<32>, 111 * 1024); if (r) return r;
    if (int lr = launch_pdl(gemm_fp8_kernel<32>, grid, dim3(320), smem, s, 0, tmW, tmX, w_scale, x_scale, (__nv_bfloat16*)y,
                            seg_off, counts, M, Nw, K, ldy, epi, splits, pipe_bytes, staging, tok_cap, scratch, tile_counters,
                            status, xs_ld)) return lr;
    return launch_result();
  }
  r = opt_in_smem(gemm_fp8_kernel<F_TOK>, 225 * 1024); if (r) return r;
  if (int lr = launch_pdl(gemm_fp8_kernel<F_TOK>, grid, dim3(320), smem, s, 0, tmW, tmX, w_scale, x_scale, (__nv_bfloat16*)y,
                          seg_off, counts, M, Nw, K, ldy, epi, splits, pipe_bytes, staging, tok_cap, scratch, tile_counters,
                          status, xs_ld)) return lr;
  return launch_result();
}

FF_EXPORT int ff_gemm_fp8(const void* xq, const float* x_scale, const void* wq, const float* w_scale, void* y,
                          const int* seg_off, const int* counts, int experts, int M, int Nw, int K, int ldy, int epi,
                          int splits, float* scratch, int* tile_counters, int* status, cudaStream_t s) {
  return gemm_fp8_launch(xq, x_scale, wq, w_scale, y, seg_off, counts, experts, M, Nw, K, ldy, epi, splits, scratch,
                         tile_counters, status, s, (long long)K, K / 128);
}

// The same with strided activations: code rows ldxq bytes apart, scale rows xs_ld floats apart (packed records
// [K codes | K / 128 scales] as they arrive from an expert-parallel dispatch: ldxq = K + K / 32, xs_ld = ldxq / 4).
FF_EXPORT int ff_gemm_fp8_strided(const void* xq, const float* x_scale, long long ldxq, int xs_ld, const void* wq,
                                  const float* w_scale, void* y, const int* seg_off, const int* counts, int experts, int M,
                                  int Nw, int K, int ldy, int epi, int* status, cudaStream_t s) {
  return gemm_fp8_launch(xq, x_scale, wq, w_scale, y, seg_off, counts, experts, M, Nw, K, ldy, epi, 1, nullptr, nullptr,
                         status, s, ldxq, xs_ld);
}
