// Decode-shape BF16 linear (M <= 256 tokens):  Y[M,N] = X[M,K] · W[N,K]ᵀ, bound by the weight
// stream from HBM, so the job of the kernel is to keep every SM pulling weights at full rate.
//
//   * Swap-AB: a 128-row weight tile is the UMMA "A" operand, the tokens are the UMMA N dimension
//     (padded to 16), so D[n (128 TMEM lanes), t (columns)] and small batches waste no tile rows.
//   * Few column tiles (tiles x 2 <= SMs): cluster split-K, the partials meet in distributed shared
//     memory (see the kernel). Otherwise:
//   * Persistent stream-K: the (column tile, k-block) work units are split evenly over one CTA per
//     SM, so no wave quantisation for any N. A CTA's share may start or end inside a tile; such
//     partial tiles go to FP32 scratch and the CTA that completes a tile (atomic arrival count)
//     adds the partials in ascending CTA order -> bitwise deterministic.
//   * Same warp-specialised pipeline as the large-M kernel (TMA producer, one MMA-issuing
//     thread, two TMEM accumulators, four epilogue warps).
//   * FUSE_AR: the tile's final sums are not stored but pushed as BF16 into every
//     tensor-parallel peer's arena slot (plain peer stores over NVLink), flagged, and the
//     rank-ordered sum of all ranks' tiles is written: the row-parallel projection and its
//     all-reduce are one kernel (no NCCL call, no second launch).
// Replaces the reference's skinny GEMM (kernels/gemm_skinny.cu: rows <= 16, 4 warps split K,
// mma.sync) and its cuBLAS calls for small row counts (src/backend/cuda/blas.rs:852-1080).
#include "ptx.cuh"
#include "comm.cuh"
#include "host_util.h"

namespace ff {

constexpr int SBM = 128;          // weight rows per tile (UMMA M)
constexpr int SBK = 64;           // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int SK_MAX_STAGES = 8;

struct alignas(8) SkinnyBars {
  uint64_t full[SK_MAX_STAGES];
  uint64_t empty[SK_MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int flag_a;
  int flag_b;
};

// CTA that owns work unit u when `total` units are split over `g` CTAs as [total*c/g, total*(c+1)/g)
__device__ __forceinline__ int unit_owner(long long u, long long total, int g) {
  return (int)(((u + 1) * g - 1) / total);
}

struct Segment { int tile, kb0, kb1; };

// iterate the segments of [u0, u1)
__device__ __forceinline__ bool next_segment(long long& u, long long u1, int kblocks, Segment& sg) {
  if (u >= u1) return false;
  sg.tile = (int)(u / kblocks);
  sg.kb0 = (int)(u - (long long)sg.tile * kblocks);
  const long long left = u1 - u;
  sg.kb1 = (int)min((long long)kblocks, sg.kb0 + left);
  u += sg.kb1 - sg.kb0;
  return true;
}

// Final output of one tile (or of this CTA's rows of it): the BF16 values sit in the staging tile
// sT[t][128]; rows handled are t = row0 + 8*row_step*i + row_step*(e/16). Either stores them to Y
// or (FUSE_AR) pushes them to every peer, waits for the peers' rows and writes the rank-ordered sum.
// Called by all 128 epilogue threads.
template <bool FUSE_AR>
__device__ __forceinline__ void emit_tile(const __nv_bfloat16* sT, __nv_bfloat16* __restrict__ Y, int M, int N, int ldy,
                                          int tile, int flag_idx, int row0, int row_step, int e, SkinnyBars& bars,
                                          const PeerArena& ar, int ar_epoch, int* status) {
  const int c16 = e & 15, r0 = e >> 4;          // 16 threads per 256-byte tile row
  const int col = tile * SBM + c16 * 8;
  const int t_first = row0 + row_step * r0, t_inc = 8 * row_step;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (!FUSE_AR) {
    const bool vec_ok = (ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0);
    if (col + 8 <= N && vec_ok) {
      for (int t = t_first; t < M; t += t_inc)
        *reinterpret_cast<uint4*>(Y + (size_t)t * ldy + col) = *reinterpret_cast<const uint4*>(sT + t * SBM + c16 * 8);
    } else if (col < N) {
      for (int t = t_first; t < M; t += t_inc)
        for (int j = 0; j < 8 && col + j < N; ++j) Y[(size_t)t * ldy + col + j] = sT[t * SBM + c16 * 8 + j];
    }
  } else {
    const int parity = ar_epoch & 1;
    if (col < N) {
      for (int pi = 1; pi < ar.world; ++pi) {
        const int p = (ar.rank + pi) % ar.world;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, p, parity, ar.rank));
        for (int t = t_first; t < M; t += t_inc)
          *reinterpret_cast<uint4*>(dst + (size_t)t * N + col) = *reinterpret_cast<const uint4*>(sT + t * SBM + c16 * 8);
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (e == 0) {
      __threadfence_system();
      for (int pi = 1; pi < ar.world; ++pi)
        st_release_sys(arena_flag(ar, (ar.rank + pi) % ar.world, ar.rank, flag_idx), ar_epoch);
      bars.flag_b = 1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (e < ar.world && e != ar.rank)
      if (!wait_flag(arena_flag(ar, ar.rank, e, flag_idx), ar_epoch, status, KID_GEMM_AR, e)) bars.flag_b = 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (bars.flag_b && col < N) {
      for (int t = t_first; t < M; t += t_inc) {
        float a8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) a8[j] = 0.f;
        for (int r = 0; r < ar.world; ++r) {
          const uint4 d = (r == ar.rank)
              ? *reinterpret_cast<const uint4*>(sT + t * SBM + c16 * 8)
              : *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const __nv_bfloat16*>(arena_slot(ar, ar.rank, parity, r)) + (size_t)t * N + col);
          const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
          for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(dp[j]); a8[2 * j] += f.x; a8[2 * j + 1] += f.y; }
        }
        uint4 o;
        o.x = pack_bf16x2(a8[0], a8[1]); o.y = pack_bf16x2(a8[2], a8[3]);
        o.z = pack_bf16x2(a8[4], a8[5]); o.w = pack_bf16x2(a8[6], a8[7]);
        *reinterpret_cast<uint4*>(Y + (size_t)t * ldy + col) = o;
      }
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");   // sT, flag_a and flag_b are reused by the next segment
}

// cl_size == 1: persistent stream-K over gridDim.x CTAs.
// cl_size  > 1: cluster split-K. Cluster c owns column tile c; its CTA r multiplies k-blocks
//   [kblocks*r/S, kblocks*(r+1)/S), leaves the FP32 partial in its own shared memory, and after a
//   cluster barrier CTA r sums token rows t = r (mod S) over the S partials through distributed shared
//   memory in CTA order (bitwise deterministic) -- no trip through global scratch, no serial fix-up.
template <bool FUSE_AR>
__global__ void __launch_bounds__(192, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   __nv_bfloat16* __restrict__ Y, int M, int N, int K, int ldy, int ntok, int stages, int stage_smem_off,
                   int cl_size, float* __restrict__ scratch, int* __restrict__ counters, int* status, PeerArena ar) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  __shared__ SkinnyBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* sT = reinterpret_cast<__nv_bfloat16*>(smem);       // BF16 staging tile [t][128]
  uint8_t* pipe = smem + stage_smem_off;
  float* sP = reinterpret_cast<float*>(pipe);                       // cluster mode: FP32 partial [t][128], after the main loop
  constexpr int A_BYTES = SBM * SBK * 2;
  const int b_bytes = ntok * SBK * 2;
  const int stage_bytes = A_BYTES + b_bytes;
  uint32_t tmem_cols = 32; while ((int)tmem_cols < 2 * ntok) tmem_cols <<= 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + SBM - 1) / SBM;
  const int kblocks = (K + SBK - 1) / SBK;
  const long long total = (long long)tiles_n * kblocks;
  const int G = gridDim.x;
  const bool clustered = cl_size > 1;
  const int crank = clustered ? (int)cluster_ctarank() : 0;
  long long u0, u1;
  if (clustered) {
    const long long base = (long long)(blockIdx.x / cl_size) * kblocks;
    u0 = base + (long long)kblocks * crank / cl_size; u1 = base + (long long)kblocks * (crank + 1) / cl_size;
  } else {
    u0 = total * blockIdx.x / G; u1 = total * (blockIdx.x + 1) / G;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0; bars.flag_a = 0; bars.flag_b = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX); }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_w = l2_policy_evict_first(), pol_x = l2_policy_evict_last();
      // Weights are written by no kernel, so the first `stages` weight tiles are requested before
      // the wait on the preceding kernel; the activations follow once that kernel is complete.
      const uint32_t pre = (uint32_t)min((long long)stages, u1 - u0);
      {
        uint32_t it = 0; long long u = u0; Segment sg;
        while (it < pre && next_segment(u, u1, kblocks, sg))
          for (int kb = sg.kb0; kb < sg.kb1 && it < pre; ++kb, ++it) {
            mbar_expect_tx(&bars.full[it], stage_bytes);
            tma_load_2d_hint(pipe + it * stage_bytes, &tmW, &bars.full[it], kb * SBK, sg.tile * SBM, pol_w);
          }
      }
      pdl_wait();
      uint32_t it = 0; bool ok = true;
      long long u = u0; Segment sg;
      while (ok && next_segment(u, u1, kblocks, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          uint8_t* sa = pipe + s * stage_bytes;
          if (it >= pre) {
            if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_SKINNY, 1)) { ok = false; break; }
            mbar_expect_tx(&bars.full[s], stage_bytes);
            tma_load_2d_hint(sa, &tmW, &bars.full[s], kb * SBK, sg.tile * SBM, pol_w);
          }
          tma_load_2d_hint(sa + A_BYTES, &tmX, &bars.full[s], kb * SBK, 0, pol_x);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(1, 1, 0, 0, SBM, ntok);
      uint32_t it = 0, seg_it = 0; bool ok = true;
      long long u = u0; Segment sg;
      while (ok && next_segment(u, u1, kblocks, sg)) {
        const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
        if (!mbar_wait(&bars.tmem_empty[acc], aph ^ 1, abort_flag, status, KID_GEMM_SKINNY, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * ntok;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_GEMM_SKINNY, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(pipe + s * stage_bytes);
          const uint64_t da = umma_desc_sw128(sa, 16, 1024);
          const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < SBK / 16; ++k) umma_f16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb > sg.kb0) || k > 0);
          umma_commit(&bars.empty[s]);
        }
        if (ok) umma_commit(&bars.tmem_full[acc]);
        ++seg_it;
      }
    }
  } else {
    // ---- epilogue warps 2..5 ; TMEM lane quarter = warp % 4 -----------------------------------
    const int q = warp & 3;
    const int nl = q * 32 + lane;                 // row inside the weight tile
    const int e = (warp - 2) * 32 + lane;         // 0..127, cooperative index
    pdl_wait();                                   // scratch, counters, the arena and Y belong to earlier kernels until here
    int ar_epoch = 0;
    if (FUSE_AR) ar_epoch = ld_volatile(arena_epoch(ar)) + 1;
    uint32_t seg_it = 0; bool ok = true;
    long long u = u0; Segment sg;
    while (ok && next_segment(u, u1, kblocks, sg)) {
      const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
      ++seg_it;
      if (!mbar_wait(&bars.tmem_full[acc], aph, abort_flag, status, KID_GEMM_SKINNY, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * ntok;
      if (clustered) {
        // the pipeline is drained (single segment): its shared memory now holds the FP32 partial
        for (int c = 0; c < ntok; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) if (c + j < M) sP[(c + j) * SBM + nl] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        break;
      }
      const bool whole = sg.kb0 == 0 && sg.kb1 == kblocks;
      bool final_here = whole;
      const int c16 = e & 15, r0 = e >> 4;          // cooperative layout: 16 threads per 256-byte tile row
      if (whole) {
        // TMEM -> BF16 staging tile sT[t][128]
        for (int c = 0; c < ntok; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) if (c + j < M) sT[(c + j) * SBM + nl] = __float2bfloat16(__uint_as_float(r[j]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
      } else {
        // partial tile: FP32 slot 2*cta + (1 if this segment starts the tile), layout [t][128]
        float* part = scratch + ((size_t)(2 * blockIdx.x + (sg.kb0 == 0 ? 1 : 0)) * M) * SBM;
        for (int c = 0; c < ntok; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) if (c + j < M) part[(size_t)(c + j) * SBM + nl] = __uint_as_float(r[j]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
        const int c_first = unit_owner((long long)sg.tile * kblocks, total, G);
        const int c_last = unit_owner((long long)(sg.tile + 1) * kblocks - 1, total, G);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e == 0) {
          const int prev = atomicAdd(&counters[sg.tile], 1);
          const int last = (prev == c_last - c_first);
          if (last) counters[sg.tile] = 0;
          bars.flag_a = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        final_here = bars.flag_a != 0;
        if (final_here) {
          __threadfence();
          // vectorised fix-up: each thread owns 8 columns of rows r0, r0+8, ...; four rows of two
          // partials at a time keep sixteen independent 16-byte loads in flight; the adds stay in
          // ascending CTA order
          for (int t0 = r0; t0 < M; t0 += 32) {
            float a[4][8];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
              for (int j = 0; j < 8; ++j) a[i][j] = 0.f;
            for (int c = c_first; c <= c_last; c += 2) {
              float4 v[2][4][2];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int cc = c + h;
                const float* src = scratch + ((size_t)(2 * cc + (cc == c_first ? 1 : 0)) * M) * SBM + c16 * 8;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int t = t0 + 8 * i;
                  if (t < M && cc <= c_last) {
                    v[h][i][0] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)t * SBM));
                    v[h][i][1] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)t * SBM + 4));
                  } else { v[h][i][0] = make_float4(0, 0, 0, 0); v[h][i][1] = v[h][i][0]; }
                }
              }
#pragma unroll
              for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  a[i][0] += v[h][i][0].x; a[i][1] += v[h][i][0].y; a[i][2] += v[h][i][0].z; a[i][3] += v[h][i][0].w;
                  a[i][4] += v[h][i][1].x; a[i][5] += v[h][i][1].y; a[i][6] += v[h][i][1].z; a[i][7] += v[h][i][1].w;
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int t = t0 + 8 * i;
              if (t < M) {
                uint4 o;
                o.x = pack_bf16x2(a[i][0], a[i][1]); o.y = pack_bf16x2(a[i][2], a[i][3]);
                o.z = pack_bf16x2(a[i][4], a[i][5]); o.w = pack_bf16x2(a[i][6], a[i][7]);
                *reinterpret_cast<uint4*>(sT + t * SBM + c16 * 8) = o;
              }
            }
          }
        }
      }
      if (final_here) emit_tile<FUSE_AR>(sT, Y, M, N, ldy, sg.tile, sg.tile, 0, 1, e, bars, ar, ar_epoch, status);
      else asm volatile("bar.sync 1, 128;" ::: "memory");   // flag_a is reused by the next segment
    }
    if (clustered) {
      // ---- cluster split-K reduction through distributed shared memory --------------------------
      __syncwarp();
      cluster_sync_all();                                      // (1) every CTA's partial is in its sP
      if (ok) {
        const int c4 = e & 31, rr = e >> 5;                    // 32 threads per FP32 row, four rows at a time
        const uint32_t sp_base = smem_u32(sP);
        for (int t = crank + cl_size * rr; t < M; t += 4 * cl_size) {
          const uint32_t off = sp_base + (uint32_t)(t * SBM + c4 * 4) * 4u;
          float4 v[8];
#pragma unroll
          for (int s = 0; s < 8; ++s) if (s < cl_size) v[s] = ld_dsmem_f4(dsmem_addr(off, s));
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int s = 0; s < 8; ++s) if (s < cl_size) { a.x += v[s].x; a.y += v[s].y; a.z += v[s].z; a.w += v[s].w; }
          uint2 o; o.x = pack_bf16x2(a.x, a.y); o.y = pack_bf16x2(a.z, a.w);
          *reinterpret_cast<uint2*>(sT + t * SBM + c4 * 4) = o;
        }
      }
      __syncwarp();
      cluster_sync_all();                                      // (2) nobody reads this CTA's sP any more
      if (ok) emit_tile<FUSE_AR>(sT, Y, M, N, ldy, sg.tile, sg.tile * cl_size + crank, crank, cl_size, e, bars, ar,
                                 ar_epoch, status);
    }
    if (FUSE_AR && e == 0) {
      __threadfence();
      const int prev = atomicAdd(arena_done(ar), 1);
      if (prev == (int)gridDim.x - 1) {
        *arena_done(ar) = 0;
        __threadfence();
        *reinterpret_cast<volatile int*>(arena_epoch(ar)) = ar_epoch;
      }
    }
  }
  if (clustered && warp < 2) {           // the producer and MMA warps take part in both cluster barriers
    __syncwarp();
    cluster_sync_all();
    cluster_sync_all();
  }

  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

}  // namespace ff
using namespace ff;

// Largest number of co-resident clusters of `s` CTAs of this kernel (0 when such a cluster cannot be
// launched); queried once per cluster size.
static int skinny_max_clusters(int s) {
  static int cached[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (s < 2 || s > 8) return 0;
  if (cached[s] >= 0) return cached[s];
  auto kern = gemm_skinny_kernel<false>;
  if (opt_in_smem(kern, 201 * 1024)) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s * 64); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = 201 * 1024;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = s; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cached[s] = n;
  return n;
}

// Cluster size for a problem (1 = persistent stream-K). Cluster split-K is used when every column
// tile can have its own co-resident cluster: few tiles, so the K range is what has to be spread
// over the SMs.
static int skinny_cluster_size(int M, int N, int K) {
  const int tiles_n = (N + SBM - 1) / SBM;
  const int kblocks = (K + SBK - 1) / SBK;
  if (M > 128 || tiles_n > 74) return 1;
  int s = 148 / tiles_n;
  if (s > 8) s = 8;
  for (; s >= 2; --s)
    if (kblocks / s >= 2 && skinny_max_clusters(s) >= tiles_n) return s;
  return 1;
}

// Plan for a problem: returns the grid size (cluster split-K: tiles x cluster size; otherwise one
// persistent CTA per SM, fewer for tiny problems);
// *scratch_bytes = FP32 partial slots (two per CTA; none in cluster mode), *counter_bytes = one int32
// per column tile (zero before the first launch; every launch leaves them zero).
FF_EXPORT int ff_gemm_skinny_plan(int M, int N, int K, long long* scratch_bytes, long long* counter_bytes) {
  const int tiles_n = (N + SBM - 1) / SBM;
  const int kblocks = (K + SBK - 1) / SBK;
  if (counter_bytes) *counter_bytes = (long long)tiles_n * 4;
  const int cl = skinny_cluster_size(M, N, K);
  if (cl > 1) {
    if (scratch_bytes) *scratch_bytes = 0;
    return tiles_n * cl;
  }
  const long long total = (long long)tiles_n * kblocks;
  long long g = total / 2;                 // at least two k-blocks of work per CTA
  if (g > 148) g = 148;
  if (g < 1) g = 1;
  if (scratch_bytes) *scratch_bytes = g > 1 ? 2 * g * (long long)M * SBM * 4 : 0;
  return (int)g;
}

template <bool FUSE_AR>
static int skinny_launch_kernel(int grid, int cl, int smem, cudaStream_t stream, const CUtensorMap& tmW,
                                const CUtensorMap& tmX, __nv_bfloat16* Y, int M, int N, int K, int ldy, int ntok,
                                int stages, int staging, float* scratch, int* counters, int* status, const PeerArena& ar) {
  auto kern = gemm_skinny_kernel<FUSE_AR>;
  static bool attr_done = false;
  if (!attr_done) { int r = opt_in_smem(kern, 201 * 1024); if (r) return r; attr_done = true; }
  return launch_pdl(kern, dim3(grid), dim3(192), smem, stream, cl, tmW, tmX, Y, M, N, K, ldy, ntok, stages, staging, cl,
                    scratch, counters, status, ar);
}

static int gemm_skinny_launch(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                              int grid, float* scratch, int* counters, int* status, cudaStream_t stream,
                              const PeerArena* arena) {
  if (M <= 0 || M > 256 || N <= 0 || K <= 0) return FF_HOST_BAD_SHAPE;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return FF_HOST_BAD_ALIGN;
  const int tiles_n = (N + SBM - 1) / SBM;
  const long long total = (long long)tiles_n * ((K + SBK - 1) / SBK);
  const int cl = skinny_cluster_size(M, N, K);
  if (cl > 1) {
    if (grid != tiles_n * cl) return FF_HOST_BAD_SHAPE;
    if (arena != nullptr && tiles_n * cl > MAX_FLAGS) return FF_HOST_TOO_LARGE;
  } else {
    if (grid < 1 || grid > 1024 || (grid > 1 && (scratch == nullptr || counters == nullptr))) return FF_HOST_BAD_SHAPE;
    if (grid > total) return FF_HOST_BAD_SHAPE;
  }
  const int ntok = (M + 15) / 16 * 16;
  CUtensorMap tmW, tmX;
  int r = make_tmap_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, (uint64_t)ldw * 2, SBK, SBM);
  if (r) return r;
  r = make_tmap_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, (uint64_t)ldx * 2, SBK, ntok);
  if (r) return r;
  const int stage_bytes = SBM * SBK * 2 + ntok * SBK * 2;
  const int staging = ((M * SBM * 2 + 1023) / 1024) * 1024;
  int stages = (200 * 1024 - staging) / stage_bytes;
  if (stages > SK_MAX_STAGES) stages = SK_MAX_STAGES;
  if (stages < 2) return FF_HOST_TOO_LARGE;
  if (cl > 1 && (long long)M * SBM * 4 > (long long)stages * stage_bytes) return FF_HOST_TOO_LARGE;
  const int smem = staging + stages * stage_bytes + 1024;
  PeerArena none = {};
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  if (arena == nullptr)
    return skinny_launch_kernel<false>(grid, cl, smem, stream, tmW, tmX, y, M, N, K, ldy, ntok, stages, staging, scratch,
                                       counters, status, none);
  return skinny_launch_kernel<true>(grid, cl, smem, stream, tmW, tmX, y, M, N, K, ldy, ntok, stages, staging, scratch,
                                    counters, status, *arena);
}

// `grid` is the value returned by ff_gemm_skinny_plan for the same problem.
FF_EXPORT int ff_gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                             int grid, float* scratch, int* counters, int* status, cudaStream_t stream) {
  return gemm_skinny_launch(X, W, Y, M, N, K, ldx, ldw, ldy, grid, scratch, counters, status, stream, nullptr);
}

// Row-parallel projection fused with the tensor-parallel all-reduce (decode shapes, M <= 256):
// Y = sum over ranks of X_r · W_rᵀ, identical bits on every rank. ptrs: arena base of every rank.
FF_EXPORT int ff_gemm_ar(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                         long long slot_bytes, const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                         int ldw, int ldy, int grid, float* scratch, int* counters, int* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return FF_HOST_BAD_SHAPE;
  if (N % 8 || (long long)M * N * 2 > slot_bytes || half_bytes < slot_bytes * world) return FF_HOST_TOO_LARGE;
  if ((N + SBM - 1) / SBM > MAX_FLAGS) return FF_HOST_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(Y) & 15) || (ldy % 8)) return FF_HOST_BAD_ALIGN;
  PeerArena a;
  for (int i = 0; i < MAX_RANKS; ++i) a.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  a.rank = rank; a.world = world; a.half_bytes = half_bytes; a.slot_bytes = slot_bytes;
  return gemm_skinny_launch(X, W, Y, M, N, K, ldx, ldw, ldy, grid, scratch, counters, status, stream, &a);
}

// ---------------------------------------------------------------------------------------
// Allocation-free variant of the decode-shape GEMM (declared in ff_noalloc.h).
//
// Some callers cannot obtain device memory at the point where they need this GEMM: code that
// runs inside a memory-budgeted plugin or a real-time serving loop whose allocator is frozen
// after start-up, or a host that simply has no allocator handle to give us (a C caller that
// only owns its input and output buffers). For them the split-K partial sums and the per-tile
// arrival counters live in a fixed array inside this library instead of caller scratch.
//
//  * Limit: the partial-sum slots (2 * grid * M * 128 * 4 bytes, grid <= 148 persistent CTAs) must
//    fit in FF_NOALLOC_SCRATCH_BYTES (8 MiB) and ceil(N/128) in FF_NOALLOC_MAX_TILES (2048); larger
//    problems are refused with FF_HOST_TOO_LARGE (in practice M <= 55 tokens for wide layers).
//    Every GPU that loads this library holds the 8 MiB until exit.
//  * The first call on a device resolves the device addresses of the arrays
//    (cudaGetSymbolAddress, with that device current) and caches them; make that first call
//    before starting any stream capture.
//  * All calls share the one array: two calls that may overlap on the GPU (different streams,
//    no ordering between them) race on it. Calls on one stream are safe. The counters are
//    cleared by every call before the kernel runs, so a call does not depend on how the
//    previous one ended.
//  * No cudaMalloc / cudaFree / allocating library routine is called here.
// ---------------------------------------------------------------------------------------
#include "ff_noalloc.h"

namespace ff {
static __device__ __align__(256) float g_noalloc_scratch[FF_NOALLOC_SCRATCH_BYTES / 4];
static __device__ __align__(256) int g_noalloc_counters[FF_NOALLOC_MAX_TILES];

struct NoAllocPtrs { float* scratch; int* counters; bool ready; };
static NoAllocPtrs g_noalloc_ptrs[64] = {};
}  // namespace ff

FF_EXPORT int ff_gemm_skinny_noalloc(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                     int ldy, int* status, cudaStream_t stream) {
  if (M <= 0 || M > 256 || N <= 0 || K <= 0) return FF_HOST_BAD_SHAPE;
  long long scratch_bytes = 0, counter_bytes = 0;
  const int grid = ff_gemm_skinny_plan(M, N, K, &scratch_bytes, &counter_bytes);
  if (scratch_bytes > (long long)FF_NOALLOC_SCRATCH_BYTES || counter_bytes > (long long)FF_NOALLOC_MAX_TILES * 4)
    return FF_HOST_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return FF_HOST_UNSUPPORTED;
  NoAllocPtrs& p = g_noalloc_ptrs[dev];
  if (!p.ready) {
    // In host code the array names are host-side stand-ins; the kernel needs the device address.
    void* ps = nullptr; void* pc = nullptr;
    e = cudaGetSymbolAddress(&ps, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaGetSymbolAddress(&pc, g_noalloc_counters);
    if (e != cudaSuccess) return static_cast<int>(e);
    p.scratch = static_cast<float*>(ps); p.counters = static_cast<int*>(pc); p.ready = true;
  }
  e = cudaMemsetAsync(p.counters, 0, (size_t)counter_bytes, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  return ff_gemm_skinny(X, W, Y, M, N, K, ldx, ldw, ldy, grid, p.scratch, p.counters, status, stream);
}
