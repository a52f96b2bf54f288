// Block-scaled FP8 (E4M3) linear on tcgen05:  Y[M,N] = dequant(Xq)[M,K] · dequant(Wq)[N,K]ᵀ
//   Wq : E4M3 codes [N,K] with one FP32 scale per 128x128 block (DeepSeek-V3 checkpoint layout)
//   Xq : E4M3 codes [M,K] with one FP32 scale per 1x128 (activation quantised by quantize.cu)
// The tensor core multiplies the raw codes (kind::f8f6f4, FP32 accumulation in TMEM) one 128-wide
// K block at a time; the epilogue warps pull each block's partial sums out of TMEM and add them
// into FP32 registers multiplied by w_scale[block] * x_scale[token, block] -- the same "per-K-block
// partial times (w_scale * x_scale)" contract as the reference's fp8_block kernels
// (kernels/fp8_linear.cu:73-140), which run on mma.sync and fall back to a BF16 materialisation +
// cuBLAS for large M. Two TMEM accumulators let block k+1 multiply while block k is promoted.
//
// Swap-AB like the BF16 decode kernel: a 128-row weight tile (exactly one scale-block row) is
// the UMMA A operand, up to 128 tokens are the UMMA N dimension. Dense use: grid (N/128, splits),
// split-K partials go through FP32 scratch and the last CTA of a tile adds them in split order.
// Grouped (MoE) use: grid (Nw/128, 1, experts) over 16-row padded expert segments, optional
// SwiGLU epilogue for gate/up weights interleaved per 64 rows.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int FBM = 128, FBK = 128, F_TOK = 128, F_STAGES_MAX = 8;

struct alignas(8) Fp8Bars {
  uint64_t full[F_STAGES_MAX];
  uint64_t empty[F_STAGES_MAX];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

__device__ __forceinline__ float silu_f8(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float bfr8(float x) { return __bfloat162float(__float2bfloat16(x)); }

// epi: 0 store, 1 SwiGLU over 64/64 interleaved rows (grouped gate/up)
__global__ void __launch_bounds__(192, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const float* __restrict__ w_scale, const float* __restrict__ x_scale, __nv_bfloat16* __restrict__ Y,
                const int* __restrict__ seg_off, const int* __restrict__ counts, int M, int Nw, int K, int ldy,
                int epi, int splits, int pipe_bytes, int stage_off, float* __restrict__ scratch,
                int* __restrict__ tile_counters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Fp8Bars bars;
  const int tn = blockIdx.x, split = blockIdx.y, e = blockIdx.z;
  const int cnt = counts ? counts[e] : M;
  if (cnt <= 0) return;
  const int row0 = seg_off ? seg_off[e] : 0;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* sT = reinterpret_cast<__nv_bfloat16*>(smem);            // [128 tok][128] bf16 = 32 KiB
  float* sXs = reinterpret_cast<float*>(smem + F_TOK * FBM * 2);         // x scales [ntok][nkb] (<= 16 KiB)
  uint8_t* pipe = smem + stage_off;
  constexpr int A_BYTES = FBM * FBK;                                     // 16 KiB of E4M3
  const int kblocks_total = (K + FBK - 1) / FBK;
  const int per = (kblocks_total + splits - 1) / splits;
  const int kb0 = split * per, kb1 = min(kblocks_total, kb0 + per);
  const int nkb = max(0, kb1 - kb0);
  const int ntok_max = min(F_TOK, ((cnt + 15) / 16) * 16);
  const int stage_bytes = A_BYTES + ntok_max * FBK;
  const int stages = min(F_STAGES_MAX, pipe_bytes / stage_bytes);
  const int chunks = (cnt + F_TOK - 1) / F_TOK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int scale_rows = (Nw + 127) / 128;                                // scale rows per expert

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0; bars.is_last = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX);
      uint32_t it = 0; bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(F_TOK, ((cnt - c * F_TOK + 15) / 16) * 16);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_FP8, 1)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], A_BYTES + ntok * FBK);
          uint8_t* sa = pipe + s * stage_bytes;
          tma_load_2d(sa, &tmW, &bars.full[s], kb * FBK, e * Nw + tn * FBM);
          for (int r = 0; r < ntok; r += 16)
            tma_load_2d(sa + A_BYTES + r * FBK, &tmX, &bars.full[s], kb * FBK, row0 + c * F_TOK + r);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, kit = 0; bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(F_TOK, ((cnt - c * F_TOK + 15) / 16) * 16);
        const uint32_t idesc = umma_idesc(0, 0, 0, 0, FBM, ntok);        // E4M3 x E4M3 -> FP32
        for (int kb = kb0; kb < kb1; ++kb, ++it, ++kit) {
          const int b = kit & 1; const uint32_t bph = (kit >> 1) & 1;
          if (!mbar_wait(&bars.tmem_empty[b], bph ^ 1, abort_flag, status, KID_GEMM_FP8, 2)) { ok = false; break; }
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_GEMM_FP8, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(pipe + s * stage_bytes);
          const uint64_t da = umma_desc_sw128(sa, 16, 1024);
          const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < FBK / 32; ++k) umma_f8f6f4(tmem_base + b * F_TOK, da + 2 * k, db + 2 * k, idesc, k != 0);
          umma_commit(&bars.empty[s]);
          umma_commit(&bars.tmem_full[b]);
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int nl = q * 32 + lane;
    const int ee = (warp - 2) * 32 + lane;
    const int n = tn * FBM + nl;
    const float* ws_row = w_scale + ((size_t)e * scale_rows + tn) * kblocks_total;
    uint32_t kit = 0; bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int ntok = min(F_TOK, ((cnt - c * F_TOK + 15) / 16) * 16);
      const int real = min(F_TOK, cnt - c * F_TOK);
      const int grow0 = row0 + c * F_TOK;
      // activation scales of this chunk and K range -> shared memory [t][nkb]
      for (int i = ee; i < ntok * nkb; i += 128) {
        const int t = i / nkb, kb = i - t * nkb;
        sXs[i] = (t < real) ? x_scale[(size_t)(grow0 + t) * kblocks_total + kb0 + kb] : 0.f;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float acc[F_TOK];
#pragma unroll
      for (int i = 0; i < F_TOK; ++i) acc[i] = 0.f;
      for (int kb = 0; kb < nkb && ok; ++kb, ++kit) {
        const int b = kit & 1; const uint32_t bph = (kit >> 1) & 1;
        if (!mbar_wait(&bars.tmem_full[b], bph, abort_flag, status, KID_GEMM_FP8, 4)) { ok = false; break; }
        tc_fence_after();
        const float ws = ws_row[kb0 + kb];
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + b * F_TOK;
#pragma unroll
        for (int cc = 0; cc < F_TOK; cc += 16) {
          if (cc < ntok) {
            uint32_t r[16];
            tmem_ld_x16(taddr + cc, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[cc + j] += __uint_as_float(r[j]) * (ws * sXs[(cc + j) * nkb + kb]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tmem_empty[b]);
      }
      if (!ok) break;
      bool final_here = true;
      if (splits > 1) {
        float* part = scratch + ((size_t)split * M) * Nw;
#pragma unroll
        for (int t = 0; t < F_TOK; ++t) if (t < real && n < Nw) part[(size_t)(grow0 + t) * Nw + n] = acc[t];
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ee == 0) {
          const int prev = atomicAdd(&tile_counters[tn * chunks + c], 1);
          bars.is_last = (prev == splits - 1);
          if (prev == splits - 1) tile_counters[tn * chunks + c] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        final_here = bars.is_last != 0;
        if (final_here) {
          __threadfence();
#pragma unroll
          for (int t = 0; t < F_TOK; ++t) {
            if (t < real) {
              float sum = 0.f;
              if (n < Nw) for (int s = 0; s < splits; ++s) sum += __ldcg(scratch + ((size_t)s * M + grow0 + t) * Nw + n);
              acc[t] = sum;
            }
          }
        }
      }
      if (final_here) {
#pragma unroll
        for (int t = 0; t < F_TOK; ++t) if (t < ntok) sT[t * FBM + nl] = __float2bfloat16(acc[t]);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi == 1) {
          const int c8 = ee & 7, r0 = ee >> 3;
          for (int t = r0; t < real; t += 16) {
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
            for (int t = r0; t < real; t += 8)
              *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t) * ldy + col) = *reinterpret_cast<const uint4*>(sT + t * FBM + c16 * 8);
          } else if (col < Nw) {
            for (int t = r0; t < real; t += 8)
              for (int j = 0; j < 8 && col + j < Nw; ++j) Y[(size_t)(grow0 + t) * ldy + col + j] = sT[t * FBM + c16 * 8 + j];
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
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
  const int chunks = (M + F_TOK - 1) / F_TOK;
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
FF_EXPORT int ff_gemm_fp8(const void* xq, const float* x_scale, const void* wq, const float* w_scale, void* y,
                          const int* seg_off, const int* counts, int experts, int M, int Nw, int K, int ldy, int epi,
                          int splits, float* scratch, int* tile_counters, int* status, cudaStream_t s) {
  if (M <= 0 || Nw <= 0 || K <= 0 || K % 128 || experts < 1) return FF_HOST_BAD_SHAPE;
  if (experts > 1 && (!seg_off || !counts || Nw % 128)) return FF_HOST_BAD_SHAPE;
  if (splits < 1 || (splits > 1 && (!scratch || !tile_counters || experts > 1))) return FF_HOST_BAD_SHAPE;
  if (epi == 1 && (Nw % 128 || ldy < Nw / 2)) return FF_HOST_BAD_SHAPE;
  if (ldy % 8 || (reinterpret_cast<uintptr_t>(y) & 15)) return FF_HOST_BAD_ALIGN;
  if ((K / 128) * F_TOK * 4 > 64 * 1024) return FF_HOST_TOO_LARGE;        // x-scale staging
  CUtensorMap tmW, tmX;
  int r = make_tmap_2d(&tmW, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, (uint64_t)experts * Nw, (uint64_t)K, FBK, FBM);
  if (r) return r;
  r = make_tmap_2d(&tmX, xq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, K, M, (uint64_t)K, FBK, 16);
  if (r) return r;
  const int staging = F_TOK * FBM * 2 + ((K / 128) * F_TOK * 4 + 1023) / 1024 * 1024;
  int pipe_bytes = 200 * 1024 - staging;
  const int smem = staging + pipe_bytes + 1024;
  r = opt_in_smem(gemm_fp8_kernel, 201 * 1024); if (r) return r;
  dim3 grid((Nw + FBM - 1) / FBM, splits, experts);
  gemm_fp8_kernel<<<grid, 192, smem, s>>>(tmW, tmX, w_scale, x_scale, (__nv_bfloat16*)y, seg_off, counts, M, Nw, K, ldy,
                                          epi, splits, pipe_bytes, staging, scratch, tile_counters, status);
  return launch_result();
}
