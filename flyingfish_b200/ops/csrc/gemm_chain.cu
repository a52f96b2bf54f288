// Decode-step projection chain: the row-parallel and column-parallel projections of a decoder
// layer and the residual-add + RMSNorm steps between them run as ONE persistent kernel.
//
// A decode step of a dense layer is  attention -> O proj -> add+norm -> gate/up (+SwiGLU) -> down ->
// add+norm -> QKV proj of the next layer (+ rotary embedding + KV-cache write). Launched one by one,
// every projection pays a fixed cost that does not shrink with the work: launch, barrier and
// tensor-memory set-up, the first weight tiles' latency, the split-K reduction tail, and no weight
// is in flight while the previous kernel drains. Here one CTA per SM keeps a single TMA -> tcgen05
// pipeline alive over all phases:
//
//   * every GEMM phase is stream-K over 128-row weight tiles (tokens on the UMMA M side, FP32
//     accumulators in TMEM, partial tiles through FP32 scratch, the CTA that completes a tile adds
//     the partials in ascending CTA order: bitwise deterministic, independent of the token count);
//   * the producer thread requests the weights of the NEXT phase as soon as pipeline stages free up
//     (weights depend on nothing), and only the activation loads wait for the previous phase: the HBM
//     stream does not stop at a phase boundary;
//   * phases are ordered by monotonic device counters instead of kernel boundaries: a GEMM phase
//     counts finished tiles, a norm phase counts finished rows; whoever needs a phase's output
//     acquire-polls its counter (bounded by a timer, like every wait in this library) and then issues
//     fence.proxy.async before TMA reads what other SMs wrote with ordinary stores;
//   * the add+norm phases are done by the epilogue warps of the CTAs that own the rows. A projection that
//     feeds a norm does not reduce its split-K partials itself: the norm gathers them (ascending CTA
//     order) while it adds the residual, which takes one synchronisation hop out of the boundary;
//   * elsewhere the CTA that arrives last at a split tile adds the other CTAs' partials to the values it
//     still holds in TMEM (again in ascending CTA order, so the bits do not depend on who is last) and
//     applies the epilogue; it never writes its own partial;
//   * publication is bar.sync + one red.release.gpu per CTA, not a fence per thread.
//
// It replaces, for decode batches of a dense GQA layer, the launch sequence of the reference's step
// (src/backend/cuda/engine.rs:2763-3330: linear, add_rmsnorm, linear, silu_mul, linear, add_rmsnorm,
// linear, rope_kv) between two attention calls.
#include "ptx.cuh"
#include "comm.cuh"
#include "host_util.h"
#include "skinny_common.cuh"

namespace ff {

constexpr int CH_MAX_PHASES = 8;
constexpr int CH_MAX_STAGES = 12;
constexpr int CH_TILE = 128;              // weight rows per tile (UMMA N)
constexpr int CH_MAX_TILES = 1024;        // per phase
constexpr int CH_THREADS = 192;
constexpr int CH_NORM_VEC = 8;            // 128 threads x 8 vectors x 8 values: hidden <= 8192
constexpr int CH_SMEM_TOTAL = 226 * 1024;  // dynamic shared memory of a CTA: pipeline stages + one FP32 staging tile

// int32 words of the synchronisation block (device memory, zero before the first launch)
constexpr int CH_SYNC_LINE = 32;                              // every polled counter has a 128-byte line of its own
constexpr int CH_SYNC_COUNT = 0;                              // [CH_MAX_PHASES] lines: units finished per phase, monotonic
constexpr int CH_SYNC_BASE = CH_MAX_PHASES * CH_SYNC_LINE;    // [CH_MAX_PHASES] value of count[] when the current launch began
constexpr int CH_SYNC_EXIT = CH_SYNC_BASE + CH_SYNC_LINE;     // CTAs that have left the current launch
constexpr int CH_SYNC_ABORT = CH_SYNC_EXIT + CH_SYNC_LINE;    // a wait ran out somewhere: everybody leaves
constexpr int CH_SYNC_WORDS = CH_SYNC_ABORT + CH_SYNC_LINE;

enum ChainKind : int { CH_GEMM = 0, CH_NORM = 1 };

struct alignas(64) ChainPhase {
  CUtensorMap tmX;              // GEMM: activations [M, K], box [ntok, 64]
  CUtensorMap tmW;              // GEMM: weights [N, K], box [128, 64]
  int kind;
  int N, K;                     // GEMM: output columns, depth.  NORM: N = hidden
  int epi;                      // GEMM: 0 store, 1 SwiGLU (Y is [M, N/2]), 2 rotary + KV write
  __nv_bfloat16* Y;             // GEMM: output.  NORM: normalised output [M, hidden]
  const __nv_bfloat16* nx;      // NORM: addend [M, hidden] (output of the preceding GEMM phase)
  __nv_bfloat16* res;           // NORM: residual stream [M, hidden], updated in place
  const __nv_bfloat16* nw;      // NORM: weight
  int ldy;
  float eps;
  int unit_offset;
  int defer;                    // GEMM: 1 = write FP32 partials only, the following norm phase gathers them
};

struct ChainParams {
  ChainPhase ph[CH_MAX_PHASES];
  SkinnyEpi rope;               // epilogue data of the phase with epi == 2
  float* scratch;               // 2 * grid slots of M * 128 FP32, chunk-major: [c/4][t] float4
  int* tile_counters;           // [CH_MAX_PHASES][2][CH_MAX_TILES] split-tile arrivals / partials written, self-resetting
  int* sync;                    // CH_SYNC_WORDS
  int* status;
  int nphase, M, ntok, stages;
  int staging_off;              // byte offset of the FP32 staging tile behind the pipeline stages
  int lookahead;                // weight stages requested before a phase's activations are known to be ready
};

struct alignas(8) ChainBars {
  uint64_t full[CH_MAX_STAGES];
  uint64_t empty[CH_MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int flag_a;
  int pad;
  float red[4];
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v; asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int atom_acq_rel_gpu_add(int* p, int v) {
  int old; asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory"); return old;
}
// ordinary (generic proxy) writes of other SMs, made visible by an acquire, become visible to TMA reads
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Bounded wait until *cnt has reached `target` (wrap-safe). Gives up when this CTA or any other has aborted.
__device__ __forceinline__ bool chain_wait(const int* cnt, int target, int* sync, volatile int* abort_s, int* status,
                                           int where) {
  if ((int)(ld_acquire_gpu(cnt) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    if ((int)(ld_acquire_gpu(cnt) - target) >= 0) return true;
    __nanosleep(32);                                  // many CTAs poll the same line: leave room for the updates
    if ((++it & 63u) == 0) {
      if (*abort_s || ld_volatile(sync + CH_SYNC_ABORT)) { *abort_s = 1; return false; }
      if (globaltimer_ns() - t0 > FF_WAIT_NS) {
        *abort_s = 1;
        atomicExch(sync + CH_SYNC_ABORT, 1);
        set_status(status, KID_CHAIN, FF_ERR_TIMEOUT, where, target);
        return false;
      }
    }
  }
}

// CTAs that take part in a GEMM phase: every one of them owns at least two (tile, k-block) units, so the owners of
// a tile's units are consecutive CTAs (the fix-up counts on that); small phases leave the other CTAs idle
__device__ __forceinline__ int phase_grid(long long total, int G) {
  long long g = total / 2;
  if (g > G) g = G;
  if (g < 1) g = 1;
  return (int)g;
}

// units a phase counts: finished tiles for a GEMM (participating CTAs when it defers its reduction), rows for a norm
__device__ __forceinline__ int phase_units(const ChainPhase& ph, int M, int G) {
  if (ph.kind != CH_GEMM) return M;
  const int tiles = (ph.N + CH_TILE - 1) / CH_TILE;
  if (!ph.defer) return tiles;
  return phase_grid((long long)tiles * ((ph.K + SBK - 1) / SBK), G);
}

__global__ void __launch_bounds__(CH_THREADS, 1)
decode_chain_kernel(const __grid_constant__ ChainParams P) {
  pdl_trigger();
  if (threadIdx.x == 0) FF_TL(P.status, KID_CHAIN, 0);
  extern __shared__ uint8_t smem_raw[];
  __shared__ ChainBars bars;
  uint8_t* pipe = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = gridDim.x;
  const int M = P.M, ntok = P.ntok, stages = P.stages;
  const int a_bytes = ntok * SBK * 2;                 // activation rows of a stage (UMMA reads 128 rows: the rest
  const int stage_bytes = a_bytes + CH_TILE * SBK * 2;   // is the stage's own weight tile, lanes never read back)
  const int tx_bytes = stage_bytes;
  constexpr uint32_t TMEM_COLS = 2 * CH_TILE;

  if (threadIdx.x == 0) {
    for (int p = 0; p < P.nphase; ++p)
      if (P.ph[p].kind == CH_GEMM) { tma_prefetch_desc(&P.ph[p].tmW); tma_prefetch_desc(&P.ph[p].tmX); }
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0; bars.flag_a = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      uint32_t it = 0; bool ok = true; bool waited_prev = false;
      for (int p = 0; p < P.nphase && ok; ++p) {
        const ChainPhase& ph = P.ph[p];
        if (ph.kind != CH_GEMM) continue;
        const int tiles = (ph.N + CH_TILE - 1) / CH_TILE;
        const int kblocks = (ph.K + SBK - 1) / SBK;
        const long long total = (long long)tiles * kblocks;
        const int gp = phase_grid(total, G);
        const bool mine = (int)blockIdx.x < gp;
        const long long u0 = mine ? total * blockIdx.x / gp : 0, u1 = mine ? total * (blockIdx.x + 1) / gp : 0;
        const int n = (int)(u1 - u0);
        const int pre = n < P.lookahead ? n : P.lookahead;
        // weights first: they depend on nothing, so they are requested while the previous phase still runs
        for (int j = 0; j < pre && ok; ++j) {
          const long long u = u0 + j;
          const int tile = (int)(u / kblocks), kb = (int)(u - (long long)tile * kblocks);
          const uint32_t idx = it + j; const int s = idx % stages; const uint32_t par = (idx / stages) & 1;
          if (idx >= (uint32_t)stages && !mbar_wait(&bars.empty[s], par ^ 1, abort_flag, P.status, KID_CHAIN, 1)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], tx_bytes);
          tma_load_2d_hint(pipe + s * stage_bytes + a_bytes, &ph.tmW, &bars.full[s], kb * SBK, tile * CH_TILE, pol_w);
        }
        if (!ok) break;
        // activations: written by the preceding kernel (first phase) or by the preceding phase
        if (!waited_prev) { pdl_wait(); waited_prev = true; }
        if (p > 0) {
          const int target = ld_volatile(P.sync + CH_SYNC_BASE + (p - 1)) + phase_units(P.ph[p - 1], M, G);
          if (!chain_wait(P.sync + CH_SYNC_COUNT + (p - 1) * CH_SYNC_LINE, target, P.sync, abort_flag, P.status, 10 + p)) { ok = false; break; }
          fence_proxy_async_global();
        }
        FF_TL(P.status, KID_CHAIN, 10 + p);
        for (int j = 0; j < pre; ++j) {
          const long long u = u0 + j;
          const int tile = (int)(u / kblocks), kb = (int)(u - (long long)tile * kblocks);
          const int s = (it + j) % stages;
          (void)tile;
          tma_load_2d_hint(pipe + s * stage_bytes, &ph.tmX, &bars.full[s], kb * SBK, 0, pol_x);
        }
        for (int j = pre; j < n; ++j) {
          const long long u = u0 + j;
          const int tile = (int)(u / kblocks), kb = (int)(u - (long long)tile * kblocks);
          const uint32_t idx = it + j; const int s = idx % stages; const uint32_t par = (idx / stages) & 1;
          if (idx >= (uint32_t)stages && !mbar_wait(&bars.empty[s], par ^ 1, abort_flag, P.status, KID_CHAIN, 2)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], tx_bytes);
          tma_load_2d_hint(pipe + s * stage_bytes + a_bytes, &ph.tmW, &bars.full[s], kb * SBK, tile * CH_TILE, pol_w);
          tma_load_2d_hint(pipe + s * stage_bytes, &ph.tmX, &bars.full[s], kb * SBK, 0, pol_x);
        }
        it += n;
        FF_TL(P.status, KID_CHAIN, 20 + p);
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(1, 1, 0, 0, STOK, CH_TILE);
      uint32_t it = 0, seg_it = 0; bool ok = true;
      for (int p = 0; p < P.nphase && ok; ++p) {
        const ChainPhase& ph = P.ph[p];
        if (ph.kind != CH_GEMM) continue;
        const int tiles = (ph.N + CH_TILE - 1) / CH_TILE;
        const int kblocks = (ph.K + SBK - 1) / SBK;
        const long long total = (long long)tiles * kblocks;
        const int gp = phase_grid(total, G);
        const bool mine = (int)blockIdx.x < gp;
        long long u = mine ? total * blockIdx.x / gp : 0; const long long u1 = mine ? total * (blockIdx.x + 1) / gp : 0;
        Segment sg;
        bool first_kb = true;
        while (ok && next_segment(u, u1, kblocks, sg)) {
          const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
          if (!mbar_wait(&bars.tmem_empty[acc], aph ^ 1, abort_flag, P.status, KID_CHAIN, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * CH_TILE;
          for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
            const int s = it % stages; const uint32_t par = (it / stages) & 1;
            if (!mbar_wait(&bars.full[s], par, abort_flag, P.status, KID_CHAIN, 4)) { ok = false; break; }
            tc_fence_after();
            if (first_kb) { FF_TL(P.status, KID_CHAIN, 30 + p); first_kb = false; }
            const uint32_t sa = smem_u32(pipe + s * stage_bytes);
            const uint64_t da = umma_desc_sw128(sa, 16, 1024);
            const uint64_t db = umma_desc_sw128(sa + a_bytes, 16, 1024);
#pragma unroll
            for (int k = 0; k < SBK / 16; ++k) umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > sg.kb0) || k > 0);
            umma_commit(&bars.empty[s]);
          }
          if (ok) umma_commit(&bars.tmem_full[acc]);
          ++seg_it;
        }
        if (mine) FF_TL(P.status, KID_CHAIN, 40 + p);
      }
    }
  } else {
    // ================================ epilogue / norm warps 2..5 ================================
    const int q = warp & 3;
    const int t_own = q * 32 + lane;              // token row held by this thread's TMEM lane
    const bool row_live = q * 32 < M;             // warp-uniform
    const int e = (warp - 2) * 32 + lane;         // 0..127
    float4* stage4 = reinterpret_cast<float4*>(pipe + P.staging_off);      // [32][M] float4, chunk-major
    pdl_wait();                                   // scratch, counters and all activations belong to earlier kernels until here
    uint32_t seg_it = 0; bool ok = true;
    const size_t slot4 = (size_t)M * (CH_TILE / 4);                        // float4 per partial slot
    for (int p = 0; p < P.nphase && ok; ++p) {
      const ChainPhase& ph = P.ph[p];
      int* done = P.sync + CH_SYNC_COUNT + p * CH_SYNC_LINE;
      if (ph.kind == CH_NORM) {
        // ---- residual add + RMSNorm of the rows this CTA owns (row r -> CTA r*G/M) ----
        const int hidden = ph.N, nvec = hidden >> 3;
        // gather mode: the addend is the sum of the preceding projection's split-K partials (rounded to BF16 as
        // the projection's output would have been), added in ascending CTA order
        const bool gather = p > 0 && P.ph[p - 1].kind == CH_GEMM && P.ph[p - 1].defer != 0;
        int g_kblocks = 1, g_gp = 1; long long g_total = 1;
        if (gather) {
          const ChainPhase& gph = P.ph[p - 1];
          g_kblocks = (gph.K + SBK - 1) / SBK;
          g_total = (long long)((gph.N + CH_TILE - 1) / CH_TILE) * g_kblocks;
          g_gp = phase_grid(g_total, G);
        }
        const float4* scr4 = reinterpret_cast<const float4*>(P.scratch);
        bool waited = false;
        for (int r = 0; r < M && ok; ++r) {
          if ((int)(((long long)r * G) / M) != (int)blockIdx.x) continue;
          if (!waited) {
            if (p > 0) {
              if (e == 0) {
                const int target = ld_volatile(P.sync + CH_SYNC_BASE + (p - 1)) + phase_units(P.ph[p - 1], M, G);
                bars.flag_a = chain_wait(P.sync + CH_SYNC_COUNT + (p - 1) * CH_SYNC_LINE, target, P.sync, abort_flag, P.status, 20 + p) ? 1 : 0;
              }
              asm volatile("bar.sync 1, 128;" ::: "memory");
              ok = bars.flag_a != 0;
              asm volatile("bar.sync 1, 128;" ::: "memory");
              if (!ok) break;
            }
            waited = true;
            if (e == 0) FF_TL(P.status, KID_CHAIN, 60 + p);
          }
          uint4 v[CH_NORM_VEC];
          // residual rows first: their latency overlaps the gather
          uint4 rr[CH_NORM_VEC];
#pragma unroll
          for (int i = 0; i < CH_NORM_VEC; ++i) {
            const int idx = e + i * 128;
            if (idx < nvec) rr[i] = __ldcg(reinterpret_cast<const uint4*>(ph.res + (size_t)r * hidden) + idx);
          }
          if (gather) {
            // four vectors of eight columns per thread and pass; per vector two partials (two float4 each) in flight
#pragma unroll
            for (int i0 = 0; i0 < CH_NORM_VEC; i0 += 4) {
              if (e + i0 * 128 >= nvec) break;
              float a8[4][8];
              int cf[4], cl[4], q0[4];
              int nmax = 0;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int idx = e + (i0 + g) * 128;
                const int tile = idx >> 4;
                q0[g] = (idx & 15) * 2;
                cf[g] = 0; cl[g] = -1;
                if (idx < nvec) {
                  cf[g] = unit_owner((long long)tile * g_kblocks, g_total, g_gp);
                  cl[g] = unit_owner((long long)(tile + 1) * g_kblocks - 1, g_total, g_gp);
                }
                nmax = max(nmax, cl[g] - cf[g] + 1);
#pragma unroll
                for (int j = 0; j < 8; ++j) a8[g][j] = 0.f;
              }
              for (int k = 0; k < nmax; k += 2) {
                float4 w4[4][2][2];
#pragma unroll
                for (int g = 0; g < 4; ++g)
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    const int cc = cf[g] + k + h;
                    if (cc <= cl[g]) {
                      const float4* src = scr4 + (size_t)(2 * cc + (cc == cf[g] ? 1 : 0)) * slot4 + (size_t)q0[g] * M + r;
                      w4[g][h][0] = __ldcg(src);
                      w4[g][h][1] = __ldcg(src + M);
                    } else { w4[g][h][0] = make_float4(0, 0, 0, 0); w4[g][h][1] = w4[g][h][0]; }
                  }
#pragma unroll
                for (int g = 0; g < 4; ++g)
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    a8[g][0] += w4[g][h][0].x; a8[g][1] += w4[g][h][0].y; a8[g][2] += w4[g][h][0].z; a8[g][3] += w4[g][h][0].w;
                    a8[g][4] += w4[g][h][1].x; a8[g][5] += w4[g][h][1].y; a8[g][6] += w4[g][h][1].z; a8[g][7] += w4[g][h][1].w;
                  }
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                v[i0 + g].x = pack_bf16x2(a8[g][0], a8[g][1]); v[i0 + g].y = pack_bf16x2(a8[g][2], a8[g][3]);
                v[i0 + g].z = pack_bf16x2(a8[g][4], a8[g][5]); v[i0 + g].w = pack_bf16x2(a8[g][6], a8[g][7]);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < CH_NORM_VEC; ++i) {
              const int idx = e + i * 128;
              if (idx < nvec) v[i] = __ldcg(reinterpret_cast<const uint4*>(ph.nx + (size_t)r * hidden) + idx);
            }
          }
          float ss = 0.f;
#pragma unroll
          for (int i = 0; i < CH_NORM_VEC; ++i) {
            const int idx = e + i * 128;
            if (idx < nvec) {
              uint32_t* ap = reinterpret_cast<uint32_t*>(&v[i]);
              const uint32_t* rp = reinterpret_cast<const uint32_t*>(&rr[i]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 fa = unpack_bf16x2(ap[j]), fr = unpack_bf16x2(rp[j]);
                ap[j] = pack_bf16x2(fa.x + fr.x, fa.y + fr.y);          // the residual is rounded to BF16 first
                const float2 f = unpack_bf16x2(ap[j]);
                ss += f.x * f.x + f.y * f.y;
              }
              reinterpret_cast<uint4*>(ph.res + (size_t)r * hidden)[idx] = v[i];
            }
          }
          ss = warp_sum(ss);
          if (lane == 0) bars.red[warp - 2] = ss;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          const float total = bars.red[0] + bars.red[1] + bars.red[2] + bars.red[3];
          const float rstd = rsqrtf(total / (float)hidden + ph.eps);
#pragma unroll
          for (int i = 0; i < CH_NORM_VEC; ++i) {
            const int idx = e + i * 128;
            if (idx < nvec) {
              const uint4 wv = reinterpret_cast<const uint4*>(ph.nw)[idx];
              const uint32_t* ap = reinterpret_cast<const uint32_t*>(&v[i]);
              const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
              uint4 o; uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float2 f = unpack_bf16x2(ap[j]), g = unpack_bf16x2(wp[j]);
                if (ph.unit_offset) { g.x += 1.f; g.y += 1.f; }
                op[j] = pack_bf16x2(f.x * rstd * g.x, f.y * rstd * g.y);
              }
              reinterpret_cast<uint4*>(ph.Y + (size_t)r * hidden)[idx] = o;
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");      // the row's stores are ordered before the release; red[] may be reused
          if (e == 0) { red_release_gpu_add(done, 1); FF_TL(P.status, KID_CHAIN, 70 + p); }
        }
        continue;
      }
      // ---- GEMM phase: this CTA's segments of the stream-K decomposition ----
      const int N = ph.N, ldy = ph.ldy;
      const int tiles = (N + CH_TILE - 1) / CH_TILE;
      const int kblocks = (ph.K + SBK - 1) / SBK;
      const long long total = (long long)tiles * kblocks;
      const int gp = phase_grid(total, G);
      const bool mine = (int)blockIdx.x < gp;
      long long u = mine ? total * blockIdx.x / gp : 0; const long long u1 = mine ? total * (blockIdx.x + 1) / gp : 0;
      int* arrive = P.tile_counters + (2 * p) * CH_MAX_TILES;
      int* written = P.tile_counters + (2 * p + 1) * CH_MAX_TILES;
      SkinnyEpi ep = P.rope; ep.mode = ph.epi;
      Segment sg;
      while (ok && next_segment(u, u1, kblocks, sg)) {
        const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
        ++seg_it;
        if (!mbar_wait(&bars.tmem_full[acc], aph, abort_flag, P.status, KID_CHAIN, 5)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * CH_TILE;
        const int col0 = sg.tile * CH_TILE;
        const bool whole = sg.kb0 == 0 && sg.kb1 == kblocks;
        float4* part4 = reinterpret_cast<float4*>(P.scratch) + (size_t)(2 * blockIdx.x + (sg.kb0 == 0 ? 1 : 0)) * slot4;
        const int c_first = whole ? (int)blockIdx.x : unit_owner((long long)sg.tile * kblocks, total, gp);
        const int c_last = whole ? (int)blockIdx.x : unit_owner((long long)(sg.tile + 1) * kblocks - 1, total, gp);
        // who finishes the tile: nobody here when the phase defers its reduction, this CTA for a whole tile, else the
        // CTA that arrives last
        bool final_here = whole && !ph.defer;
        if (!whole && !ph.defer) {
          if (e == 0) {
            const int prev = atom_acq_rel_gpu_add(&arrive[sg.tile], 1);
            const int last = (prev == c_last - c_first);
            if (last) arrive[sg.tile] = 0;
            bars.flag_a = last;
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          final_here = bars.flag_a != 0;
          asm volatile("bar.sync 1, 128;" ::: "memory");     // flag_a may be rewritten below
        }
        if (whole && final_here) {
          // ---- a whole tile: TMEM -> registers -> epilogue -> output ----
          if (row_live && ph.epi != 0) {
            for (int c = 0; c < 64; c += 16) {
              uint32_t gq[16], uq[16];
              tmem_ld_x16(taddr + c, gq);
              tmem_ld_x16(taddr + 64 + c, uq);
              tmem_ld_wait();
              if (t_own < M) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
                  emit_pair(ep, ph.Y, N, ldy, t_own, sg.tile, (c >> 3) + h, reinterpret_cast<const float*>(gq) + 8 * h,
                            reinterpret_cast<const float*>(uq) + 8 * h, P.status);
              }
            }
          } else if (row_live) {
            for (int c = 0; c < CH_TILE; c += 16) {
              uint32_t r[16];
              tmem_ld_x16(taddr + c, r);
              tmem_ld_wait();
              if (t_own < M) {
                uint4 o0, o1;
                o0.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])); o0.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                o0.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])); o0.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                o1.x = pack_bf16x2(__uint_as_float(r[8]), __uint_as_float(r[9])); o1.y = pack_bf16x2(__uint_as_float(r[10]), __uint_as_float(r[11]));
                o1.z = pack_bf16x2(__uint_as_float(r[12]), __uint_as_float(r[13])); o1.w = pack_bf16x2(__uint_as_float(r[14]), __uint_as_float(r[15]));
                uint4* dst = reinterpret_cast<uint4*>(ph.Y + (size_t)t_own * ldy + col0 + c);
                dst[0] = o0; dst[1] = o1;
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (e == 0) red_release_gpu_add(done, 1);
          continue;
        }
        // ---- a piece of a tile: FP32 values leave TMEM chunk-major ([c/4][t] float4: a warp's accesses are contiguous),
        // to global scratch, or to the staging tile in shared memory when this CTA finishes the tile ----
        {
          float4* dst4 = final_here ? stage4 : part4;
          if (row_live) {
            for (int c = 0; c < CH_TILE; c += 16) {
              uint32_t r[16];
              tmem_ld_x16(taddr + c, r);
              tmem_ld_wait();
              if (t_own < M) {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  dst4[(size_t)((c >> 2) + j) * M + t_own] =
                      make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                  __uint_as_float(r[4 * j + 3]));
              }
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
        }
        if (!final_here) {
          if (!ph.defer) {
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (e == 0) red_release_gpu_add(&written[sg.tile], 1);
          }
          continue;
        }
        // ---- last to arrive at a split tile: wait for the other pieces, add all in ascending CTA order ----
        if (e == 0) {
          const int okw = chain_wait(&written[sg.tile], c_last - c_first, P.sync, abort_flag, P.status, 30 + p) ? 1 : 0;
          if (okw) written[sg.tile] = 0;
          bars.flag_a = okw;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");         // also: the staging tile is complete
        ok = bars.flag_a != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!ok) break;
        {
          const float4* scr4 = reinterpret_cast<const float4*>(P.scratch);
          const bool paired = ph.epi != 0;
          // item: (j8, t) with t fastest; paired mode takes chunks j8 and j8 + 8 of a row together
          const int items = paired ? 8 * M : 16 * M;
          for (int i0 = e; i0 < items; i0 += (paired ? 256 : 512)) {
            float a8[4][8];
            int tq[4], qq[4];      // row and first float4 chunk of each of the four vectors handled at a time
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int it_ = paired ? i0 + 128 * (g >> 1) : i0 + 128 * g;
              const int j8 = it_ / M;
              tq[g] = it_ < items ? it_ - j8 * M : -1;
              qq[g] = 2 * (paired ? j8 + 8 * (g & 1) : j8);
#pragma unroll
              for (int j = 0; j < 8; ++j) a8[g][j] = 0.f;
            }
            for (int c = c_first; c <= c_last; c += 2) {
              float4 w4[4][2][2];
#pragma unroll
              for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  const int cc = c + h;
                  if (tq[g] >= 0 && cc <= c_last) {
                    const size_t off = (size_t)qq[g] * M + tq[g];
                    if (cc == (int)blockIdx.x) {
                      w4[g][h][0] = stage4[off]; w4[g][h][1] = stage4[off + M];
                    } else {
                      const float4* src = scr4 + (size_t)(2 * cc + (cc == c_first ? 1 : 0)) * slot4 + off;
                      w4[g][h][0] = __ldcg(src); w4[g][h][1] = __ldcg(src + M);
                    }
                  } else { w4[g][h][0] = make_float4(0, 0, 0, 0); w4[g][h][1] = w4[g][h][0]; }
                }
#pragma unroll
              for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  a8[g][0] += w4[g][h][0].x; a8[g][1] += w4[g][h][0].y; a8[g][2] += w4[g][h][0].z; a8[g][3] += w4[g][h][0].w;
                  a8[g][4] += w4[g][h][1].x; a8[g][5] += w4[g][h][1].y; a8[g][6] += w4[g][h][1].z; a8[g][7] += w4[g][h][1].w;
                }
            }
            if (paired) {
#pragma unroll
              for (int g = 0; g < 4; g += 2)
                if (tq[g] >= 0) emit_pair(ep, ph.Y, N, ldy, tq[g], sg.tile, qq[g] >> 1, a8[g], a8[g + 1], P.status);
            } else {
#pragma unroll
              for (int g = 0; g < 4; ++g)
                if (tq[g] >= 0) {
                  uint4 o;
                  o.x = pack_bf16x2(a8[g][0], a8[g][1]); o.y = pack_bf16x2(a8[g][2], a8[g][3]);
                  o.z = pack_bf16x2(a8[g][4], a8[g][5]); o.w = pack_bf16x2(a8[g][6], a8[g][7]);
                  *reinterpret_cast<uint4*>(ph.Y + (size_t)tq[g] * ldy + col0 + (qq[g] >> 1) * 8) = o;
                }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");         // the tile is stored; the staging tile may be reused
        if (e == 0) red_release_gpu_add(done, 1);
      }
      if (ok && ph.defer && mine) {
        // all pieces of this CTA are written: one release per CTA
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e == 0) red_release_gpu_add(done, 1);
      }
      if (mine && e == 0) FF_TL(P.status, KID_CHAIN, 50 + p);
    }
  }

  __syncthreads();
  if (threadIdx.x == 0) FF_TL(P.status, KID_CHAIN, 99);
  if (bars.abort_flag) {
    if (threadIdx.x == 0) atomicExch(P.sync + CH_SYNC_ABORT, 1);
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }    // copies in flight may still land in shared memory
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (threadIdx.x == 0) {
    // the last CTA to leave moves the bases up to the counters' values of a complete launch
    __threadfence();
    const int prev = atomicAdd(P.sync + CH_SYNC_EXIT, 1);
    if (prev == G - 1) {
      if (ld_volatile(P.sync + CH_SYNC_ABORT) == 0)
        for (int p = 0; p < P.nphase; ++p) P.sync[CH_SYNC_BASE + p] += phase_units(P.ph[p], M, G);
      P.sync[CH_SYNC_EXIT] = 0;
      __threadfence();
    }
  }
}

}  // namespace ff
using namespace ff;

// One phase of a chain as the host describes it (mirrored by ctypes in ops/chain.py).
struct FFChainPhase {
  int kind;                 // 0 GEMM, 1 add + RMSNorm
  int epi;                  // GEMM: 0 store, 1 SwiGLU, 2 rotary + KV write
  int N, K;                 // GEMM: output columns and depth (epi 1: N counts the interleaved gate/up rows). NORM: N = hidden
  const void* X; int ldx;   // GEMM: activations [M, K]
  const void* W; int ldw;   // GEMM: weights [N, K]
  void* Y; int ldy;         // GEMM: output. NORM: normalised output [M, hidden]
  const void* nx;           // NORM: addend [M, hidden]
  void* res;                // NORM: residual [M, hidden], in place
  const void* nw;           // NORM: weight [hidden]
  float eps; int unit_offset;
};

struct FFChainRope {
  const float* cos_sin; const int* slots; void* kcache; void* vcache;
  int hq, hkv, rot_dim, block_size, num_blocks;
};

// Bytes of FP32 scratch and of int32 tile counters / synchronisation words a chain of `M` rows needs
// (the same buffers serve every launch on a stream; all must be zero before the first one).
FF_EXPORT int ff_decode_chain_workspace(int M, long long* scratch_bytes, long long* counter_bytes, long long* sync_bytes) {
  if (M <= 0 || M > STOK) return FF_HOST_BAD_SHAPE;
  if (scratch_bytes) *scratch_bytes = 2ll * sm_count() * M * CH_TILE * 4;
  if (counter_bytes) *counter_bytes = 2ll * CH_MAX_PHASES * CH_MAX_TILES * 4;
  if (sync_bytes) *sync_bytes = CH_SYNC_WORDS * 4;
  return 0;
}

FF_EXPORT int ff_decode_chain(const FFChainPhase* phases, int nphase, int M, const FFChainRope* rope, float* scratch,
                              int* tile_counters, int* sync, int* status, cudaStream_t stream) {
  if (phases == nullptr || nphase < 1 || nphase > CH_MAX_PHASES || M <= 0 || M > STOK) return FF_HOST_BAD_SHAPE;
  if (scratch == nullptr || tile_counters == nullptr || sync == nullptr) return FF_HOST_BAD_SHAPE;
  ChainParams P = {};
  P.nphase = nphase; P.M = M; P.ntok = (M + 15) / 16 * 16;
  const int staging = M * CH_TILE * 4;                                    // FP32 tile of the CTA that finishes a split tile
  P.stages = (CH_SMEM_TOTAL - 1024 - staging) / ((P.ntok + CH_TILE) * SBK * 2);
  if (P.stages > CH_MAX_STAGES) P.stages = CH_MAX_STAGES;
  if (P.stages < 2) return FF_HOST_TOO_LARGE;
  P.staging_off = P.stages * (P.ntok + CH_TILE) * SBK * 2;
  P.lookahead = P.stages;
  if (const char* ev = getenv("FF_CHAIN_LOOKAHEAD")) { const int v = atoi(ev); if (v >= 1 && v < P.stages) P.lookahead = v; }
  P.scratch = scratch; P.tile_counters = tile_counters; P.sync = sync; P.status = status;
  bool any_gemm = false;
  for (int p = 0; p < nphase; ++p) {
    const FFChainPhase& h = phases[p];
    ChainPhase& d = P.ph[p];
    d.kind = h.kind; d.N = h.N; d.K = h.K; d.epi = h.epi; d.ldy = h.ldy; d.eps = h.eps; d.unit_offset = h.unit_offset;
    d.Y = static_cast<__nv_bfloat16*>(h.Y);
    if (h.kind == CH_GEMM) {
      any_gemm = true;
      if (h.N <= 0 || h.K <= 0 || (h.N % CH_TILE) || (h.K % 8) || (h.ldx % 8) || (h.ldw % 8) || (h.ldy % 8)) return FF_HOST_BAD_SHAPE;
      if (h.N / CH_TILE > CH_MAX_TILES) return FF_HOST_TOO_LARGE;
      if (h.epi < 0 || h.epi > 2 || (reinterpret_cast<uintptr_t>(h.Y) & 15)) return FF_HOST_BAD_ALIGN;
      if (h.epi == 2) {
        if (rope == nullptr || rope->hq <= 0 || rope->hkv <= 0 || h.N != (rope->hq + 2 * rope->hkv) * 128 ||
            rope->rot_dim > 128 || (rope->rot_dim % 2)) return FF_HOST_BAD_SHAPE;
      }
      int r = make_tmap_2d(&d.tmX, h.X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, h.K, M, (uint64_t)h.ldx * 2, SBK, P.ntok);
      if (r) return r;
      r = make_tmap_2d(&d.tmW, h.W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, h.K, h.N, (uint64_t)h.ldw * 2, SBK, CH_TILE);
      if (r) return r;
    } else if (h.kind == CH_NORM) {
      if (h.N <= 0 || (h.N % 8) || h.N > 128 * 8 * CH_NORM_VEC) return FF_HOST_BAD_SHAPE;
      if (h.nx == nullptr || h.res == nullptr || h.nw == nullptr || h.Y == nullptr) return FF_HOST_BAD_SHAPE;
      if ((reinterpret_cast<uintptr_t>(h.nx) | reinterpret_cast<uintptr_t>(h.res) | reinterpret_cast<uintptr_t>(h.nw) |
           reinterpret_cast<uintptr_t>(h.Y)) & 15) return FF_HOST_BAD_ALIGN;
      d.nx = static_cast<const __nv_bfloat16*>(h.nx); d.res = static_cast<__nv_bfloat16*>(h.res);
      d.nw = static_cast<const __nv_bfloat16*>(h.nw);
    } else {
      return FF_HOST_BAD_SHAPE;
    }
  }
  if (!any_gemm) return FF_HOST_BAD_SHAPE;
  // A projection whose output only feeds the norm that follows leaves its split-K reduction to that norm, provided no
  // CTA holds more than two pieces (its share of the units is no longer than a tile's k-blocks).
  static const bool defer_on = [] { const char* ev = getenv("FF_CHAIN_DEFER"); return !(ev && ev[0] == '0'); }();
  for (int p = 0; p + 1 < nphase; ++p) {
    ChainPhase& d = P.ph[p];
    const ChainPhase& nx = P.ph[p + 1];
    if (!defer_on || d.kind != CH_GEMM || d.epi != 0 || nx.kind != CH_NORM || nx.nx != d.Y || nx.N != d.N) continue;
    const long long kblocks = (d.K + SBK - 1) / SBK, total = (long long)(d.N / CH_TILE) * kblocks;
    long long gp = total / 2; if (gp > sm_count()) gp = sm_count(); if (gp < 1) gp = 1;
    if ((total + gp - 1) / gp <= kblocks && gp > 1) d.defer = 1;
  }
  if (rope != nullptr) {
    P.rope.mode = 2; P.rope.cos_sin = reinterpret_cast<const float2*>(rope->cos_sin); P.rope.slots = rope->slots;
    P.rope.kcache = static_cast<__nv_bfloat16*>(rope->kcache); P.rope.vcache = static_cast<__nv_bfloat16*>(rope->vcache);
    P.rope.hq = rope->hq; P.rope.hkv = rope->hkv; P.rope.rot_dim = rope->rot_dim; P.rope.block_size = rope->block_size;
    P.rope.num_blocks = rope->num_blocks;
  }
  const int smem = P.staging_off + staging + 1024;
  if (int r = opt_in_smem(decode_chain_kernel, CH_SMEM_TOTAL)) return r;
  // one CTA per SM: every CTA must be resident for the phase counters to advance
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_chain_kernel, CH_THREADS, smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return FF_HOST_UNSUPPORTED;
  }
  return launch_pdl(decode_chain_kernel, dim3(sm_count()), dim3(CH_THREADS), smem, stream, 0, P);
}
