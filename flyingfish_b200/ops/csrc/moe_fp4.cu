// Grouped expert GEMM over NVFP4 weights without a BF16 copy of them in memory (W4A16):
//   Y[seg rows, Nw] = Xs[seg rows, K] · (e2m1(Wq[e]) * e4m3(Wsc[e]) * global[e])[Nw, K]ᵀ
// Wq  : [E_local * Nw, K / 2] bytes, two E2M1 codes per byte, low nibble first
// Wsc : [E_local * Nw, K / 16] bytes, one E4M3 scale per 16 weights
// global : FP32 per expert (ModelOpt `weight_scale_2`)
// The decode-sized MoE layer is bound by expert weight bytes, so the weights stay packed in HBM (a quarter of the
// BF16 bytes) and are expanded on the way into the tensor-core operand:
//   * four converter warps read the packed codes of a 128-row x 128-wide K block (a warp-wide load covers eight
//     whole 64-byte row pieces) and its scales straight from global memory, two K blocks ahead in registers,
//     expand them to BF16 (byte-permute look-ups in registers, four codes at a time, one BF16x2 multiply by the
//     group's scale; e2m1 * e4m3 is exact in BF16: 2 + 4 significant bits) and write the two 64-wide
//     128-byte-swizzled sub-tiles that tcgen05.mma reads as its A operand;
//   * one thread streams the tokens of the segment (the UMMA N side, up to 32 per pass) with TMA;
//   * one thread issues the MMAs into a TMEM accumulator; the per-expert global scale is applied in FP32 in the
//     epilogue (more exact than folding it into a BF16 weight), with the optional SwiGLU of gate/up stacks
//     interleaved per 64 rows. Two CTAs share an SM (97 KiB of shared memory, <= 168 registers), so one CTA's
//     prologue, pipeline fill and epilogue overlap the other's main loop.
// Swap-AB like the BF16 grouped kernel of moe.cu (weights = UMMA M, tokens = UMMA N). Segments longer than 32 tokens
// are processed in passes of 32 that each re-expand the weights, so this kernel is meant for decode-sized segments;
// prefill-sized calls expand the weights once (quantize.cu) and use the tiled grouped GEMM.
// Format: kernels/nvfp4_linear.cu and src/fp8.rs:124-147 of the reference.
#include "ptx.cuh"
#include "host_util.h"
#include <cuda_fp8.h>

namespace ff {

constexpr int F4_BM = 128;           // weight rows per CTA (UMMA M)
constexpr int F4_KB = 128;           // K per pipeline stage = two 64-wide UMMA sub-tiles
constexpr int F4_NSUB = F4_KB / 64;
constexpr int F4_TOK = 32;           // tokens per pass (UMMA N)
constexpr int F4_STAGES = 2;
constexpr int F4_SUB = F4_BM * 64 * 2;               // one converted sub-tile: 16 KiB
constexpr int F4_A_BYTES = F4_NSUB * F4_SUB;         // 32 KiB
constexpr int F4_X_BYTES = F4_NSUB * F4_TOK * 128;   // 8 KiB
constexpr int F4_STAGE_BYTES = F4_A_BYTES + F4_X_BYTES;
constexpr int F4_EPI_TOK = 32;
constexpr int F4_STAGING = F4_EPI_TOK * F4_BM * 4;   // FP32 transpose tile of the epilogue: 16 KiB

struct alignas(8) Fp4Bars {
  uint64_t full[F4_STAGES];
  uint64_t empty[F4_STAGES];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float f4_silu(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float f4_bfr(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ float f4_e4m3(uint32_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
// E2M1 code -> value: sign | 2-bit exponent | 1-bit mantissa; magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
__device__ __forceinline__ float f4_value(uint32_t code) {
  const uint32_t m = code & 7u;
  // exponent field 0: 0 or 0.5 (subnormal); otherwise (1 + man / 2) * 2^(exp - 1)
  const float mag = (m < 2u) ? 0.5f * (float)m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
  return (code & 8u) ? -mag : mag;
}

// grid (Nw / 128, E_local), 192 threads: warp 0 token TMA, warp 1 MMA, warps 2..5 converters + epilogue
__global__ void __launch_bounds__(192, 2)
moe_fp4_grouped_kernel(const __grid_constant__ CUtensorMap tmX, const uint8_t* __restrict__ Wq,
                       const uint8_t* __restrict__ Wsc, const float* __restrict__ Wglobal, __nv_bfloat16* __restrict__ Y,
                       const int* __restrict__ seg_off, const int* __restrict__ counts, int Nw, int K, int ldy, int epi,
                       int* status, int capacity) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Fp4Bars bars;
  const int e = blockIdx.y, tn = blockIdx.x;
  // a segment reaching past the row buffers (an overflowed dispatch, reported through the status word) is cut there
  const int cnt = min(counts[e], capacity - seg_off[e]);
  if (cnt <= 0) return;                                   // uniform for the CTA
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sT = reinterpret_cast<float*>(smem);             // epilogue staging [32 tokens][128] fp32
  uint8_t* pipe = smem + F4_STAGING;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = seg_off[e];
  const int kblocks = K / F4_KB;
  const int passes = (cnt + F4_TOK - 1) / F4_TOK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < F4_STAGES; ++i) { mbar_init(&bars.full[i], 5); mbar_init(&bars.empty[i], 1); }
    mbar_init(&bars.tmem_full, 1); mbar_init(&bars.tmem_empty, 4);
    bars.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmX);
      uint32_t it = 0; bool ok = true;
      for (int p = 0; p < passes && ok; ++p) {
        const int ntok = min(F4_TOK, ((cnt - p * F4_TOK + 15) / 16) * 16);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % F4_STAGES; const uint32_t ph = (it / F4_STAGES) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_MOE_GEMM, 11)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], F4_NSUB * ntok * 128);
          uint8_t* sx = pipe + s * F4_STAGE_BYTES + F4_A_BYTES;
          for (int j = 0; j < F4_NSUB; ++j)
            for (int r = 0; r < ntok; r += 16)
              tma_load_2d(sx + j * (F4_TOK * 128) + r * 128, &tmX, &bars.full[s], kb * F4_KB + j * 64,
                          row0 + p * F4_TOK + r);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0; bool ok = true;
      for (int p = 0; p < passes && ok; ++p) {
        const int ntok = min(F4_TOK, ((cnt - p * F4_TOK + 15) / 16) * 16);
        const uint32_t idesc = umma_idesc(1, 1, 0, 0, F4_BM, ntok);
        if (!mbar_wait(&bars.tmem_empty, (p & 1) ^ 1, abort_flag, status, KID_MOE_GEMM, 12)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % F4_STAGES; const uint32_t ph = (it / F4_STAGES) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_MOE_GEMM, 13)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(pipe + s * F4_STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < F4_NSUB; ++j) {
            const uint64_t da = umma_desc_sw128(sa + j * F4_SUB, 16, 1024);
            const uint64_t db = umma_desc_sw128(sa + F4_A_BYTES + j * (F4_TOK * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | j | k) != 0);
          }
          umma_commit(&bars.empty[s]);
        }
        if (ok) umma_commit(&bars.tmem_full);
      }
    }
  } else {
    // ---- converter + epilogue warps. Converter warp cw owns weight rows cw*32 .. cw*32+31 of the tile; load i of
    // a K block gives lane l the 16 packed bytes (32 weights) of chunk l%4 of row cw*32 + i*8 + l/4, so a warp-wide
    // load covers eight whole 64-byte row pieces. ------------------------------------------------------------------
    const int wr = threadIdx.x - 64;                                    // 0..127 (epilogue indexing)
    const int q = warp & 3;                                             // TMEM lane quarter of this warp
    const int cw = warp - 2, pc = lane & 3;
    const size_t grow = (size_t)e * Nw + (size_t)tn * F4_BM + cw * 32 + (lane >> 2);
    const uint8_t* wq = Wq + grow * (size_t)(K / 2) + pc * 16;
    const uint8_t* ws = Wsc + grow * (size_t)(K / 16) + pc * 2;
    const size_t wq_step = (size_t)8 * (K / 2), ws_step = (size_t)8 * (K / 16);      // eight rows further per load
    const float gscale = Wglobal[e];
    const int total = passes * kblocks;
    // register prefetch, two K blocks ahead (two named register sets: no dynamic indexing)
    uint4 pk0[4], pk1[4];
    uint32_t sc0[4], sc1[4];
    auto fetch = [&](uint4 (&pk)[4], uint32_t (&sc)[4], int it) {
      const int kb = it % kblocks;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pk[i] = __ldg(reinterpret_cast<const uint4*>(wq + i * wq_step + (size_t)kb * (F4_KB / 2)));
        sc[i] = __ldg(reinterpret_cast<const unsigned short*>(ws + i * ws_step + (size_t)kb * (F4_KB / 16)));
      }
    };
    // 8 codes of a 32-bit word -> four BF16 pairs times the group's scale (exact in BF16). The magnitude of a code
    // indexes two 8-entry byte tables (high and low byte of the BF16 value) held in registers: prmt looks up four
    // codes at once, two more prmt interleave the bytes into BF16 pairs, the sign bits are moved into place.
    auto expand4 = [&](uint32_t w, __nv_bfloat162 sv) -> uint4 {
      const uint32_t mag = w & 0x77777777u;
      const uint32_t hi_a = __byte_perm(0x3f3f3f00u, 0x40404040u, mag);            // codes 0..3: high bytes
      const uint32_t lo_a = __byte_perm(0xc0800000u, 0xc0804000u, mag);            //             low bytes
      const uint32_t hi_b = __byte_perm(0x3f3f3f00u, 0x40404040u, mag >> 16);      // codes 4..7
      const uint32_t lo_b = __byte_perm(0xc0800000u, 0xc0804000u, mag >> 16);
      uint32_t o[4];
      o[0] = __byte_perm(lo_a, hi_a, 0x5140) | ((w & 0x00000008u) << 12) | ((w & 0x00000080u) << 24);
      o[1] = __byte_perm(lo_a, hi_a, 0x7362) | ((w & 0x00000800u) << 4) | ((w & 0x00008000u) << 16);
      o[2] = __byte_perm(lo_b, hi_b, 0x5140) | ((w & 0x00080000u) >> 4) | ((w & 0x00800000u) << 8);
      o[3] = __byte_perm(lo_b, hi_b, 0x7362) | ((w & 0x08000000u) >> 12) | (w & 0x80000000u);
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) {
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&o[b2]), sv);
        o[b2] = *reinterpret_cast<const uint32_t*>(&r);
      }
      return make_uint4(o[0], o[1], o[2], o[3]);
    };
    auto convert = [&](const uint4 (&pk)[4], const uint32_t (&sc)[4], uint8_t* stage) {
      uint8_t* sub = stage + (pc >> 1) * F4_SUB;                        // 64 weights of a row = one sub-tile row
      const int ch0 = (pc & 1) * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = cw * 32 + i * 8 + (lane >> 2);
        const __nv_bfloat162 s0 = __float2bfloat162_rn(f4_e4m3(sc[i] & 0xffu));
        const __nv_bfloat162 s1 = __float2bfloat162_rn(f4_e4m3(sc[i] >> 8));
        uint8_t* rowp = sub + r * 128;
        const int x = r & 7;
        *reinterpret_cast<uint4*>(rowp + (((ch0 + 0) ^ x) << 4)) = expand4(pk[i].x, s0);
        *reinterpret_cast<uint4*>(rowp + (((ch0 + 1) ^ x) << 4)) = expand4(pk[i].y, s0);
        *reinterpret_cast<uint4*>(rowp + (((ch0 + 2) ^ x) << 4)) = expand4(pk[i].z, s1);
        *reinterpret_cast<uint4*>(rowp + (((ch0 + 3) ^ x) << 4)) = expand4(pk[i].w, s1);
      }
    };
    fetch(pk0, sc0, 0);
    if (total > 1) fetch(pk1, sc1, 1);
    bool ok = true;
    int it = 0;
    for (int p = 0; p < passes && ok; ++p) {
      const int ntok = min(F4_TOK, ((cnt - p * F4_TOK + 15) / 16) * 16);
      const int real = min(F4_TOK, cnt - p * F4_TOK);
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % F4_STAGES; const uint32_t ph = (it / F4_STAGES) & 1;
        if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_MOE_GEMM, 14)) { ok = false; break; }
        uint8_t* sa = pipe + s * F4_STAGE_BYTES;
        if (it & 1) { convert(pk1, sc1, sa); if (it + 2 < total) fetch(pk1, sc1, it + 2); }
        else        { convert(pk0, sc0, sa); if (it + 2 < total) fetch(pk0, sc0, it + 2); }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.full[s]);
      }
      if (!ok) break;
      // ---- epilogue of this pass --------------------------------------------------------------------
      if (!mbar_wait(&bars.tmem_full, p & 1, abort_flag, status, KID_MOE_GEMM, 15)) { ok = false; break; }
      tc_fence_after();
      const int nl = q * 32 + lane;                                     // accumulator lane = weight row of the tile
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
      const int grow0 = row0 + p * F4_TOK;
      for (int t0 = 0; t0 < ntok; t0 += F4_EPI_TOK) {                   // the FP32 transpose tile holds 32 tokens
        const int tcount = min(F4_EPI_TOK, ntok - t0);
        for (int cc = 0; cc < tcount; cc += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + t0 + cc, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) sT[(cc + j) * F4_BM + nl] = __uint_as_float(r[j]) * gscale;
        }
        if (t0 + F4_EPI_TOK >= ntok) {                                  // accumulator fully read: the next pass may start
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.tmem_empty);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (epi == 1) {
          const int c8 = wr & 7, r0 = wr >> 3;                          // 16 token rows per sweep, 8 outputs per thread
          for (int t = r0; t < tcount; t += 16) {
            if (t0 + t >= real) break;
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = c8 * 8 + 2 * j;
              const float g0 = f4_bfr(sT[t * F4_BM + col]), g1 = f4_bfr(sT[t * F4_BM + col + 1]);
              const float u0 = f4_bfr(sT[t * F4_BM + 64 + col]), u1 = f4_bfr(sT[t * F4_BM + 64 + col + 1]);
              o[j] = pack_bf16x2(f4_bfr(f4_silu(g0)) * u0, f4_bfr(f4_silu(g1)) * u1);
            }
            *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t0 + t) * ldy + tn * 64 + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        } else {
          const int c16 = wr & 15, r0 = wr >> 4;                        // 8 token rows per sweep
          for (int t = r0; t < tcount; t += 8) {
            if (t0 + t >= real) break;
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(sT[t * F4_BM + c16 * 8 + 2 * j], sT[t * F4_BM + c16 * 8 + 2 * j + 1]);
            *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t0 + t) * ldy + tn * F4_BM + c16 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
  }
  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 64); }
}

}  // namespace ff
using namespace ff;

// Xs [capacity, K] bf16 sorted token rows; Wq / Wsc / Wglobal as described at the top; Y [capacity, ldy] bf16.
// epi 0: Y has Nw columns; epi 1: SwiGLU of gate/up rows interleaved per 64, Y has Nw / 2 columns.
FF_EXPORT int ff_moe_grouped_gemm_nvfp4(const void* xs, const void* wq, const void* wsc, const float* wglobal, void* y,
                                        const int* seg_off, const int* counts, int E_local, int Nw, int K, int capacity,
                                        int ldy, int epi, int* status, cudaStream_t s) {
  if (E_local <= 0 || Nw <= 0 || K <= 0 || capacity <= 0 || !seg_off || !counts || !wglobal) return FF_HOST_BAD_SHAPE;
  if (Nw % F4_BM || K % F4_KB || (epi != 0 && epi != 1)) return FF_HOST_BAD_SHAPE;
  if (ldy % 8 || ldy < (epi == 1 ? Nw / 2 : Nw)) return FF_HOST_BAD_ALIGN;
  if ((reinterpret_cast<uintptr_t>(wq) & 15) || (reinterpret_cast<uintptr_t>(wsc) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15)) return FF_HOST_BAD_ALIGN;
  CUtensorMap tmX;
  int r = make_tmap_2d(&tmX, xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, capacity, (uint64_t)K * 2, 64, 16);
  if (r) return r;
  const int smem = F4_STAGING + F4_STAGES * F4_STAGE_BYTES + 1024;
  r = opt_in_smem(moe_fp4_grouped_kernel, smem); if (r) return r;
  dim3 grid(Nw / F4_BM, E_local);
  moe_fp4_grouped_kernel<<<grid, 192, smem, s>>>(tmX, (const uint8_t*)wq, (const uint8_t*)wsc, wglobal, (__nv_bfloat16*)y,
                                                 seg_off, counts, Nw, K, ldy, epi, status, capacity);
  return launch_result();
}
