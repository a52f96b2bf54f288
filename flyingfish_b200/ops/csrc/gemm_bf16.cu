// BF16 linear layers on 5th-generation tensor cores:  Y[M,N] = X[M,K] · W[N,K]ᵀ
// (activations row-major, weights in the checkpoint's [out, in] layout, FP32 accumulation,
// one BF16 rounding at the end).
//
// Two kernels share one warp-specialised pipeline (TMA producer warp -> mbarrier ring ->
// single-thread tcgen05.mma issuer -> TMEM accumulator -> 4 epilogue warps):
//   * gemm_bf16_kernel   : M >= 128-ish. Persistent, 128 x BN x 64 tiles, double-buffered
//                          TMEM accumulators so the epilogue of tile i overlaps the mainloop
//                          of tile i+1. Optional fused SwiGLU epilogue (gate|up interleaved
//                          per 128 columns in the weight).
//   * gemm_skinny_kernel : decode shapes (M <= 256). Swap-AB: the weight tile is the 128-row
//                          UMMA "A" operand and the tokens are the UMMA N dimension, so a
//                          16-token batch does not waste a 128-row tile; split-K with a
//                          deterministic in-kernel fix-up (last CTA of a column tile sums the
//                          FP32 partials in split order) spreads the weight stream over all SMs.
// This replaces the reference's cuBLAS/cuBLASLt calls (src/backend/cuda/blas.rs:852-1080)
// and its mma.sync skinny kernel (kernels/gemm_skinny.cu).
#include "ptx.cuh"
#include "comm.cuh"
#include "host_util.h"

namespace ff {

constexpr int BM = 128;
constexpr int BK = 64;           // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;

struct alignas(8) PipeBars {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int is_last;
};

// grouped raster: GROUP_M row-tiles share a band of column tiles so both operands stay in L2
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(tiles_m - first_m, GROUP_M);
  const int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// epi: 0 = store bf16; 1 = SwiGLU (columns [0,BN/2) of a tile are gate, [BN/2,BN) are up; output
// has N/2 columns); 2 = store fp32.
template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 void* __restrict__ Cout, int M, int N, int K, int ldc, int epi, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;   // 256 or 512, power of two
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES; const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_BF16, 1)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], STAGE_BYTES);
          uint8_t* sa = smem + s * STAGE_BYTES;
          tma_load_2d(sa, &tmA, &bars.full[s], kb * BK, tm * BM);
          tma_load_2d(sa + A_BYTES, &tmB, &bars.full[s], kb * BK, tn * BN);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1, 1, 0, 0, BM, BN);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
        const int acc = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
        if (!mbar_wait(&bars.tmem_empty[acc], aph ^ 1, abort_flag, status, KID_GEMM_BF16, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES; const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_GEMM_BF16, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(sa, 16, 1024);
          const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +32 bytes per K step inside the 128-byte swizzle row = +2 in the address field
            umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(&bars.empty[s]);
        }
        if (ok) umma_commit(&bars.tmem_full[acc]);
      }
    }
  } else {
    // epilogue warps 2..5 ; TMEM lane quarter = warp % 4
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_it) {
      int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
      const int acc = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
      if (!mbar_wait(&bars.tmem_full[acc], aph, abort_flag, status, KID_GEMM_BF16, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      if (epi == 1) {
        constexpr int HALF = BN / 2;
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + (size_t)row * ldc + (size_t)tn * HALF;
        const int ncols_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 16) {
          uint32_t g[16], u[16];
          tmem_ld_x16(taddr + c, g);
          tmem_ld_x16(taddr + HALF + c, u);
          tmem_ld_wait();
          if (row < M) {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
              const float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
              // rounding policy "mode 0" of the reference's silu_mul (kernels/act.cu:220-262):
              // gate and up are BF16 values, silu rounded to BF16, product rounded again.
              const float a0 = __bfloat162float(__float2bfloat16(silu_f(__bfloat162float(__float2bfloat16(g0)))));
              const float a1 = __bfloat162float(__float2bfloat16(silu_f(__bfloat162float(__float2bfloat16(g1)))));
              o[j] = pack_bf16x2(a0 * __bfloat162float(__float2bfloat16(u0)),
                                 a1 * __bfloat162float(__float2bfloat16(u1)));
            }
            if (tn * HALF + c + 16 <= ncols_out) {
              uint4* dst = reinterpret_cast<uint4*>(crow + c);
              dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
              dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
            } else {
              for (int j = 0; j < 16; ++j)
                if (tn * HALF + c + j < ncols_out) {
                  const uint32_t w = o[j >> 1];
                  reinterpret_cast<uint16_t*>(crow + c)[j] = (j & 1) ? uint16_t(w >> 16) : uint16_t(w & 0xffff);
                }
            }
          }
        }
      } else if (epi == 2) {
        float* crow = reinterpret_cast<float*>(Cout) + (size_t)row * ldc + (size_t)tn * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
          if (row < M) {
            if (tn * BN + c + 16 <= N) {
              uint4* dst = reinterpret_cast<uint4*>(crow + c);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
            } else {
              for (int j = 0; j < 16; ++j) if (tn * BN + c + j < N) crow[c + j] = __uint_as_float(r[j]);
            }
          }
        }
      } else {
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + (size_t)row * ldc + (size_t)tn * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_x32(taddr + c, r);
          tmem_ld_wait();
          if (row < M) {
            if (tn * BN + c + 32 <= N) {
              uint4* dst = reinterpret_cast<uint4*>(crow + c);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                dst[j] = make_uint4(pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                                    pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (tn * BN + c + j < N) crow[c + j] = __float2bfloat16(__uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
    }
  }

  // teardown: every thread arrives here, also after a timed-out wait
  __syncthreads();
  if (bars.abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}


}  // namespace ff

using namespace ff;

// Y[M,N] = X[M,K] · W[N,K]ᵀ. epi: 0 bf16 out, 1 fused SwiGLU (out has N/2 columns), 2 fp32 out.
// ldx / ldw / ldy in elements. Returns 0 or an error code (see host_util.h).
FF_EXPORT int ff_gemm_bf16(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                           int epi, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return FF_HOST_BAD_SHAPE;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return FF_HOST_BAD_ALIGN;
  if (epi == 1 && (N % 256)) return FF_HOST_BAD_SHAPE;
  const int out_cols = (epi == 1) ? N / 2 : N;
  const int out_bytes = (epi == 2) ? 4 : 2;
  if (((size_t)ldy * out_bytes) % 16 || ldy < out_cols) return FF_HOST_BAD_ALIGN;
  if (reinterpret_cast<uintptr_t>(Y) & 15) return FF_HOST_BAD_ALIGN;
  CUtensorMap tmA, tmB;
  constexpr int BN = 256, STAGES = 4;
  int r = make_tmap_2d(&tmA, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, (uint64_t)ldx * 2, BK, BM);
  if (r) return r;
  r = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, (uint64_t)ldw * 2, BK, BN);
  if (r) return r;
  const int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto kern = gemm_bf16_kernel<BN, STAGES>;
  static bool attr_done = false;
  if (!attr_done) { r = opt_in_smem(kern, smem); if (r) return r; attr_done = true; }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 192, smem, stream>>>(tmA, tmB, Y, M, N, K, ldy, epi, status);
  return launch_result();
}

