// Decode-shape BF16 linear (M <= 128 tokens):  Y[M,N] = X[M,K] · W[N,K]ᵀ, bound by the weight
// stream from HBM, so the job of the kernel is to keep every SM pulling weights at full rate.
//
//   * The tokens are the UMMA M dimension (128 TMEM lanes, only ceil16(M) rows are loaded, the rest of
//     the accumulator is never read) and up to 256 weight rows are the UMMA N dimension. A
//     tcgen05.mma costs about the same whatever its N, so the weight bytes one instruction consumes
//     decide how fast an SM can stream: with the weights as the wide B operand (256 rows x 32 bytes per
//     instruction) the tensor pipe is no longer the limit; with the weights as the 128-row A operand
//     (swap-AB) it capped an SM near 40 GB/s, below its share of HBM.
//   * Few weight tiles: cluster split-K. One cluster per tile of `tile_rows` weight rows, CTA s of
//     the cluster multiplies its share of K and pushes the FP32 partial of token rows t = r (mod S)
//     into slot s of CTA r's shared memory (distributed-shared-memory stores); after one cluster
//     barrier every CTA sums its rows over the S slots in CTA order (bitwise deterministic) from its
//     own shared memory: no global scratch, no serial fix-up, no remote loads. tile_rows (a multiple of 16, at most 256) is chosen so that tiles x S fills the SMs.
//   * Many tiles: persistent stream-K. The (tile, k-block) units are split evenly over one CTA per SM;
//     partial tiles go to FP32 scratch and the CTA that completes a tile (arrival counter) adds the
//     partials in ascending CTA order -> bitwise deterministic.
//   * Warp-specialised pipeline (TMA producer, one MMA-issuing thread, two TMEM accumulators, four
//     epilogue warps). Launched with programmatic dependent launch: barriers, TMEM and the first
//     weight tiles are set up while the preceding kernel still runs; activations are read after
//     griddepcontrol.wait.
//   * FUSE_AR: the final sums are not stored but written as BF16 into every tensor-parallel rank's
//     arena slot (plain peer stores over NVLink, own slot included), flagged, and the rank-ordered
//     sum of all ranks' values is written: the row-parallel projection and its all-reduce are one
//     kernel (no NCCL call, no second launch).
// Replaces the reference's skinny GEMM (kernels/gemm_skinny.cu: rows <= 16, 4 warps split K,
// mma.sync) and its cuBLAS calls for small row counts (src/backend/cuda/blas.rs:852-1080).
#include "ptx.cuh"
#include "comm.cuh"
#include "host_util.h"
#include <mutex>
#include <vector>
#include "skinny_common.cuh"

namespace ff {

constexpr int SK_MAX_STAGES = 8;
constexpr int SP_PAD = 4;         // FP32 partial rows in shared memory are padded by 4 floats

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

// Where the final values of a tile go: Y, or (FUSE_AR) the arena slot of this rank on every rank.
template <bool FUSE_AR>
struct TileSink {
  __nv_bfloat16* Y; int N, ldy; bool vec8;      // vec8: 16-byte stores of eight values are aligned
  PeerArena ar; int parity;

  // eight consecutive columns col..col+7 of token row t (col is a multiple of 8)
  __device__ __forceinline__ void put8(int t, int col, const float* a) const {
    if (col >= N) return;
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]); o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]); o.w = pack_bf16x2(a[6], a[7]);
    if (!FUSE_AR) {
      __nv_bfloat16* dst = Y + (size_t)t * ldy + col;
      if (vec8 && col + 8 <= N) { *reinterpret_cast<uint4*>(dst) = o; return; }
      const __nv_bfloat16* ob = reinterpret_cast<const __nv_bfloat16*>(&o);
      for (int j = 0; j < 8 && col + j < N; ++j) dst[j] = ob[j];
    } else {
      // N % 8 == 0 and 16-byte aligned slots are checked by the host
      if (ar.mc_base != nullptr && ar.mc_oneshot) {
        // NVLS one-shot: ONE multicast store puts the contribution into this rank's slot on every rank
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, ar.rank, parity, ar.rank)) + (size_t)t * N + col;
        multimem_st_bf16x8(arena_mc(ar, dst), o);
        return;
      }
      if (ar.mc_base != nullptr) {
        // NVLS: the contribution stays in this rank's own slot 0; the switch sums the ranks' copies
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, ar.rank, parity, 0)) + (size_t)t * N + col;
        *reinterpret_cast<uint4*>(dst) = o;
        return;
      }
      for (int pi = 0; pi < ar.world; ++pi) {
        const int p = (ar.rank + pi) % ar.world;
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, p, parity, ar.rank)) + (size_t)t * N + col;
        *reinterpret_cast<uint4*>(dst) = o;
      }
    }
  }
};

// FUSE_AR: after this CTA's values of (tile, rows row0 + i*row_step) are in every rank's slot, flag the
// peers, wait for theirs, and write the rank-ordered sum. Called by all 128 epilogue threads.
__device__ __forceinline__ void allreduce_tile(const TileSink<true>& sink, int M, int tile, int tile_rows, int flag_idx,
                                               int row0, int row_step, int e, SkinnyBars& bars, int ar_epoch, int* status) {
  const PeerArena& ar = sink.ar;
  if (ar.mc_base != nullptr && !ar.mc_oneshot) {
    // ---- NVLS two-shot: every rank flags its contribution on all ranks with one multicast store; the owner of
    // this chunk (flag_idx % world) lets the switch sum the ranks' copies (multimem.ld_reduce, FP32 accumulate) and
    // multicasts the BF16 result into slot 1 of every rank, then flags it; every rank copies its result to Y.
    // One rank reduces a chunk, so all ranks see the same bits.
    const int owner = flag_idx % ar.world;
    const int vec_per_row = tile_rows / 8;
    const int rows = (M - row0 + row_step - 1) / row_step;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (e == 0) {
      __threadfence_system();
      multimem_st_release(arena_mc(ar, arena_flag(ar, ar.rank, ar.rank, flag_idx)), ar_epoch);
      bars.flag_b = 1;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (ar.rank == owner) {
      if (e < ar.world && e != ar.rank)
        if (!wait_flag(arena_flag(ar, ar.rank, e, flag_idx), ar_epoch, status, KID_GEMM_AR, e)) bars.flag_b = 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (bars.flag_b) {
        for (int i = e; i < rows * vec_per_row; i += 128) {
          const int t = row0 + (i / vec_per_row) * row_step;
          const int col = tile * tile_rows + (i % vec_per_row) * 8;
          if (col >= sink.N) continue;
          const size_t off = (size_t)t * sink.N + col;
          __nv_bfloat16* src = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, ar.rank, sink.parity, 0)) + off;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ar, ar.rank, sink.parity, 1)) + off;
          multimem_st_bf16x8(arena_mc(ar, dst), multimem_ld_reduce_bf16x8(arena_mc(ar, src)));
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (e == 0 && bars.flag_b) {
        __threadfence_system();
        multimem_st_release(arena_mc(ar, arena_flag(ar, ar.rank, ar.rank, flag_idx + MAX_FLAGS / 2)), ar_epoch);
      }
    }
    if (e == 0)
      if (!wait_flag(arena_flag(ar, ar.rank, owner, flag_idx + MAX_FLAGS / 2), ar_epoch, status, KID_GEMM_AR, 100 + owner)) bars.flag_b = 0;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (bars.flag_b) {
      for (int i = e; i < rows * vec_per_row; i += 128) {
        const int t = row0 + (i / vec_per_row) * row_step;
        const int col = tile * tile_rows + (i % vec_per_row) * 8;
        if (col >= sink.N) continue;
        // written by the owner's multicast store: read past L1
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(arena_slot(ar, ar.rank, sink.parity, 1)) + (size_t)t * sink.N + col));
        *reinterpret_cast<uint4*>(sink.Y + (size_t)t * sink.ldy + col) = v;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // flag_b is reused by the next tile
    return;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (e == 0) {
    __threadfence_system();
    if (ar.mc_base != nullptr) {
      // NVLS one-shot: one release store flags every rank (the data went out as multicast stores too)
      multimem_st_release(arena_mc(ar, arena_flag(ar, ar.rank, ar.rank, flag_idx)), ar_epoch);
    } else {
      for (int pi = 1; pi < ar.world; ++pi)
        st_release_sys(arena_flag(ar, (ar.rank + pi) % ar.world, ar.rank, flag_idx), ar_epoch);
    }
    bars.flag_b = 1;
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");
  // with multicast stores this rank's own copy also travels through the switch: its flag is waited for like a peer's
  if (e < ar.world && (e != ar.rank || ar.mc_base != nullptr))
    if (!wait_flag(arena_flag(ar, ar.rank, e, flag_idx), ar_epoch, status, KID_GEMM_AR, e)) bars.flag_b = 0;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (bars.flag_b) {
    const int vec_per_row = tile_rows / 8;                       // 16-byte vectors of eight values
    const int rows = (M - row0 + row_step - 1) / row_step;
    for (int i = e; i < rows * vec_per_row; i += 128) {
      const int t = row0 + (i / vec_per_row) * row_step;
      const int col = tile * tile_rows + (i % vec_per_row) * 8;
      if (col >= sink.N) continue;
      float a8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a8[j] = 0.f;
      for (int r = 0; r < ar.world; ++r) {
        const uint4 d = *reinterpret_cast<const uint4*>(
            reinterpret_cast<const __nv_bfloat16*>(arena_slot(ar, ar.rank, sink.parity, r)) + (size_t)t * sink.N + col);
        const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(dp[j]); a8[2 * j] += f.x; a8[2 * j + 1] += f.y; }
      }
      uint4 o;
      o.x = pack_bf16x2(a8[0], a8[1]); o.y = pack_bf16x2(a8[2], a8[3]);
      o.z = pack_bf16x2(a8[4], a8[5]); o.w = pack_bf16x2(a8[6], a8[7]);
      *reinterpret_cast<uint4*>(sink.Y + (size_t)t * sink.ldy + col) = o;
    }
  }
  asm volatile("bar.sync 1, 128;" ::: "memory");   // flag_b is reused by the next tile
}

// cl_size == 1: persistent stream-K over gridDim.x CTAs.  cl_size > 1: cluster split-K, cluster c
// owns weight tile c, CTA r of it the k-blocks [kblocks*r/S, kblocks*(r+1)/S).
template <bool FUSE_AR>
__global__ void __launch_bounds__(192, 2)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   __nv_bfloat16* __restrict__ Y, int M, int N, int K, int ldy, int ntok, int tile_rows, int stages,
                   int cl_size, int pipe_off, float* __restrict__ scratch, int* __restrict__ counters, int* status,
                   PeerArena ar, SkinnyEpi ep) {
  pdl_trigger();
  if (cl_size > 1) cluster_arrive_relaxed();         // phase A: "this CTA runs" (waited on before the first remote store)
  if (threadIdx.x == 0) FF_TL(status, KID_GEMM_SKINNY, 0);
  extern __shared__ uint8_t smem_raw[];
  __shared__ SkinnyBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // cluster mode: receive buffer [source CTA][owned row][tile_rows + SP_PAD] FP32 for the partials of this CTA's rows
  float* recv = reinterpret_cast<float*>(smem);
  uint8_t* pipe = smem + pipe_off;
  // activation rows of a stage: only the ntok loaded rows take space; the UMMA reads 128 rows, i.e. on into the
  // stage's own weight tile (and the next stage; the launcher leaves slack behind the last one), and those
  // accumulator lanes are never read back
  const int A_BYTES = ntok * SBK * 2;
  const int stage_bytes = A_BYTES + tile_rows * SBK * 2;
  const int tx_bytes = (ntok + tile_rows) * SBK * 2;
  uint32_t tmem_cols = 32; while ((int)tmem_cols < 2 * tile_rows) tmem_cols <<= 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (N + tile_rows - 1) / tile_rows;
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

  // Thread 0 is the TMA producer. It initialises the barriers and at once requests the first `stages`
  // weight tiles (weights are written by no kernel, so this needs no wait on the preceding kernel),
  // while warp 1 allocates TMEM; the other roles meet it at the block barrier.
  const uint32_t pre = (uint32_t)min((long long)stages, u1 - u0);
  uint64_t pol_w = 0;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX);
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0; bars.flag_a = 0; bars.flag_b = 0;
    mbar_fence_init();
    pol_w = l2_policy_evict_first();
    uint32_t it = 0; long long u = u0; Segment sg;
    while (it < pre && next_segment(u, u1, kblocks, sg))
      for (int kb = sg.kb0; kb < sg.kb1 && it < pre; ++kb, ++it) {
        mbar_expect_tx(&bars.full[it], tx_bytes);
        tma_load_2d_hint(pipe + it * stage_bytes + A_BYTES, &tmW, &bars.full[it], kb * SBK, sg.tile * tile_rows, pol_w);
      }
    FF_TL(status, KID_GEMM_SKINNY, 2);
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, tmem_cols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;
  if (threadIdx.x == 0) FF_TL(status, KID_GEMM_SKINNY, 1);

  if (warp == 0) {
    if (lane == 0) {
      const uint64_t pol_x = l2_policy_evict_last();
      pdl_wait();
      FF_TL(status, KID_GEMM_SKINNY, 3);
      uint32_t it = 0; bool ok = true;
      long long u = u0; Segment sg;
      while (ok && next_segment(u, u1, kblocks, sg)) {
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          uint8_t* sa = pipe + s * stage_bytes;
          if (it >= pre) {
            if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_SKINNY, 1)) { ok = false; break; }
            mbar_expect_tx(&bars.full[s], tx_bytes);
            tma_load_2d_hint(sa + A_BYTES, &tmW, &bars.full[s], kb * SBK, sg.tile * tile_rows, pol_w);
          }
          tma_load_2d_hint(sa, &tmX, &bars.full[s], kb * SBK, 0, pol_x);
        }
      }
      FF_TL(status, KID_GEMM_SKINNY, 4);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(1, 1, 0, 0, STOK, tile_rows);
      uint32_t it = 0, seg_it = 0; bool ok = true;
      long long u = u0; Segment sg;
      while (ok && next_segment(u, u1, kblocks, sg)) {
        const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
        if (!mbar_wait(&bars.tmem_empty[acc], aph ^ 1, abort_flag, status, KID_GEMM_SKINNY, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * tile_rows;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_GEMM_SKINNY, 3)) { ok = false; break; }
          tc_fence_after();
          if (it == 0) FF_TL(status, KID_GEMM_SKINNY, 5);
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
      FF_TL(status, KID_GEMM_SKINNY, 6);
    }
  } else {
    // ---- epilogue warps 2..5 ; TMEM lane quarter = warp % 4 ; lane = token ----------------------
    const int q = warp & 3;
    const int t_own = q * 32 + lane;              // token row held by this thread's TMEM lane
    const bool row_live = q * 32 < M;             // warp-uniform: this quarter holds real tokens
    const int e = (warp - 2) * 32 + lane;         // 0..127, cooperative index
    const int vpr = tile_rows / 8;                // 8-value vectors per tile row
    pdl_wait();                                   // scratch, counters, the arena and Y belong to earlier kernels until here
    if (e == 0) FF_TL(status, KID_GEMM_SKINNY, 7);
    int ar_epoch = 0;
    if (FUSE_AR) ar_epoch = ld_volatile(arena_epoch(ar)) + 1;
    TileSink<FUSE_AR> sink;
    sink.Y = Y; sink.N = N; sink.ldy = ldy; sink.ar = ar; sink.parity = ar_epoch & 1;
    sink.vec8 = FUSE_AR || ((ldy % 8 == 0) && ((reinterpret_cast<uintptr_t>(Y) & 15) == 0));
    uint32_t seg_it = 0; bool ok = true;
    long long u = u0; Segment sg;
    sg.tile = 0; sg.kb0 = 0; sg.kb1 = 0;
    while (ok && next_segment(u, u1, kblocks, sg)) {
      const int acc = seg_it & 1; const uint32_t aph = (seg_it >> 1) & 1;
      ++seg_it;
      if (!mbar_wait(&bars.tmem_full[acc], aph, abort_flag, status, KID_GEMM_SKINNY, 4)) { ok = false; break; }
      tc_fence_after();
      if (e == 0) FF_TL(status, KID_GEMM_SKINNY, 8);
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * tile_rows;
      const int col0 = sg.tile * tile_rows;
      if (clustered) {
        // push this CTA's partial of token row t into slot `crank` of the row's owner, CTA t % S
        cluster_wait();                                          // phase A: every CTA of the cluster runs
        if (row_live) {
          const int rows_per = (M + cl_size - 1) / cl_size;
          const int owner = t_own % cl_size, ti = t_own / cl_size;
          const uint32_t dst = dsmem_addr(
              smem_u32(recv) + (uint32_t)((crank * rows_per + ti) * (tile_rows + SP_PAD)) * 4u, owner);
          for (int c = 0; c < tile_rows; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(taddr + c, r);
            tmem_ld_wait();
            if (t_own < M) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                st_dsmem_f4(dst + (uint32_t)(c + 4 * j) * 4u,
                            make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                        __uint_as_float(r[4 * j + 3])));
            }
          }
        }
        tc_fence_before();
        break;
      }
      const bool whole = sg.kb0 == 0 && sg.kb1 == kblocks;
      if (whole) {
        // TMEM -> registers -> output
        if (row_live && ep.mode != 0) {
          for (int c = 0; c < 64; c += 16) {
            uint32_t g[16], u[16];
            tmem_ld_x16(taddr + c, g);
            tmem_ld_x16(taddr + 64 + c, u);
            tmem_ld_wait();
            if (t_own < M) {
#pragma unroll
              for (int h = 0; h < 2; ++h)
                emit_pair(ep, Y, N, ldy, t_own, sg.tile, (c >> 3) + h, reinterpret_cast<const float*>(g) + 8 * h,
                          reinterpret_cast<const float*>(u) + 8 * h, status);
            }
          }
        } else if (row_live) {
          for (int c = 0; c < tile_rows; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(taddr + c, r);
            tmem_ld_wait();
            if (t_own < M) {
              float a8[8];
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 8; ++j) a8[j] = __uint_as_float(r[8 * h + j]);
                sink.put8(t_own, col0 + c + 8 * h, a8);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars.tmem_empty[acc]);
        if constexpr (FUSE_AR) allreduce_tile(sink, M, sg.tile, tile_rows, sg.tile, 0, 1, e, bars, ar_epoch, status);
        continue;
      }
      // partial tile: FP32 slot 2*cta + (1 if this segment starts the tile), layout [t][tile_rows]
      const size_t slot_elems = (size_t)M * tile_rows;
      float* part = scratch + (size_t)(2 * blockIdx.x + (sg.kb0 == 0 ? 1 : 0)) * slot_elems;
      if (row_live && t_own < M)      // single-writer contract of the partial slots: one claim per (slot, token row)
        dbg_write_once(status, KID_GEMM_SKINNY, DBG_GEMM_PARTIAL, (long long)(2 * blockIdx.x + (sg.kb0 == 0 ? 1 : 0)) * M + t_own);
      if (row_live) {
        for (int c = 0; c < tile_rows; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + c, r);
          tmem_ld_wait();
          if (t_own < M) {
            float4* dst = reinterpret_cast<float4*>(part + (size_t)t_own * tile_rows + c);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                                   __uint_as_float(r[4 * j + 3]));
          }
        }
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
      const bool final_here = bars.flag_a != 0;
      if (final_here) {
        __threadfence();
        // fix-up: 8-value vectors of the tile are dealt round-robin to the 128 threads; four vectors of two
        // partials (sixteen independent 16-byte loads) are in flight at a time; the adds stay in ascending
        // CTA order
        // with a row-wise epilogue a thread takes the two paired vectors (j8, j8 + 8) of a row together
        const bool paired = ep.mode != 0;
        const int nvec = M * vpr;
        const int i_end = paired ? M * 8 : nvec;
        for (int i0 = e; i0 < i_end; i0 += (paired ? 256 : 512)) {
          float a8[4][8];
#pragma unroll
          for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) a8[g][j] = 0.f;
          for (int c = c_first; c <= c_last; c += 2) {
            float4 v[4][2][2];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              int i = i0 + 128 * g;
              if (paired) { const int pr = i0 + 128 * (g >> 1); i = pr < i_end ? (pr >> 3) * 16 + (pr & 7) + 8 * (g & 1) : nvec; }
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int cc = c + h;
                if (i < nvec && cc <= c_last) {
                  const float* src = scratch + (size_t)(2 * cc + (cc == c_first ? 1 : 0)) * slot_elems + (size_t)i * 8;
                  v[g][h][0] = __ldcg(reinterpret_cast<const float4*>(src));
                  v[g][h][1] = __ldcg(reinterpret_cast<const float4*>(src + 4));
                } else { v[g][h][0] = make_float4(0, 0, 0, 0); v[g][h][1] = v[g][h][0]; }
              }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                a8[g][0] += v[g][h][0].x; a8[g][1] += v[g][h][0].y; a8[g][2] += v[g][h][0].z; a8[g][3] += v[g][h][0].w;
                a8[g][4] += v[g][h][1].x; a8[g][5] += v[g][h][1].y; a8[g][6] += v[g][h][1].z; a8[g][7] += v[g][h][1].w;
              }
          }
          if (paired) {
#pragma unroll
            for (int g = 0; g < 4; g += 2) {
              const int pr = i0 + 128 * (g >> 1);
              if (pr < i_end) emit_pair(ep, Y, N, ldy, pr >> 3, sg.tile, pr & 7, a8[g], a8[g + 1], status);
            }
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int i = i0 + 128 * g;
              if (i < nvec) { const int t = i / vpr, c8 = i - t * vpr; sink.put8(t, col0 + c8 * 8, a8[g]); }
            }
          }
        }
        if constexpr (FUSE_AR) allreduce_tile(sink, M, sg.tile, tile_rows, sg.tile, 0, 1, e, bars, ar_epoch, status);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // flag_a is reused by the next segment
    }
    if (clustered) {
      // ---- cluster split-K reduction: every partial of this CTA's rows is in its receive buffer after
      // the barrier; nothing touches another CTA's shared memory afterwards, so CTAs leave independently
      if (!ok) cluster_wait();                                 // phase A was not consumed on the error path
      __syncwarp();
      cluster_sync_all();                                      // phase B
      if (e == 0) FF_TL(status, KID_GEMM_SKINNY, 9);
      if (ok) {
        const int rows_per = (M + cl_size - 1) / cl_size;
        const int rows = (M - crank + cl_size - 1) / cl_size;  // token rows t = crank (mod cl_size)
        const int col0 = sg.tile * tile_rows;
        const int ldp = tile_rows + SP_PAD;
        if (ep.mode != 0) {
          for (int i = e; i < rows * 8; i += 128) {
            const int ti = i >> 3, j8 = i & 7;
            float lo[8], hi[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { lo[j] = 0.f; hi[j] = 0.f; }
            for (int s = 0; s < cl_size; ++s) {
              const float4* p4 = reinterpret_cast<const float4*>(recv + ((size_t)s * rows_per + ti) * ldp + j8 * 8);
              const float4 l0 = p4[0], l1 = p4[1], h0 = p4[16], h1 = p4[17];
              lo[0] += l0.x; lo[1] += l0.y; lo[2] += l0.z; lo[3] += l0.w; lo[4] += l1.x; lo[5] += l1.y; lo[6] += l1.z; lo[7] += l1.w;
              hi[0] += h0.x; hi[1] += h0.y; hi[2] += h0.z; hi[3] += h0.w; hi[4] += h1.x; hi[5] += h1.y; hi[6] += h1.z; hi[7] += h1.w;
            }
            emit_pair(ep, Y, N, ldy, crank + ti * cl_size, sg.tile, j8, lo, hi, status);
          }
        } else
        for (int i = e; i < rows * vpr; i += 128) {
          const int ti = i / vpr, c8 = i - ti * vpr;
          const float* src = recv + (size_t)ti * ldp + c8 * 8;
          float4 v[8][2];
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s < cl_size) {
              const float4* p4 = reinterpret_cast<const float4*>(src + (size_t)s * rows_per * ldp);
              v[s][0] = p4[0]; v[s][1] = p4[1];
            }
          float a8[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) a8[j] = 0.f;
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s < cl_size) {
              a8[0] += v[s][0].x; a8[1] += v[s][0].y; a8[2] += v[s][0].z; a8[3] += v[s][0].w;
              a8[4] += v[s][1].x; a8[5] += v[s][1].y; a8[6] += v[s][1].z; a8[7] += v[s][1].w;
            }
          sink.put8(crank + ti * cl_size, col0 + c8 * 8, a8);
        }
      }
      if constexpr (FUSE_AR)
        if (ok) allreduce_tile(sink, M, sg.tile, tile_rows, sg.tile * cl_size + crank, crank, cl_size, e, bars, ar_epoch, status);
    }
    if (e == 0) FF_TL(status, KID_GEMM_SKINNY, 10);
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
  if (clustered && warp < 2) {           // the producer and MMA warps take part in both cluster barrier phases
    __syncwarp();
    cluster_wait();
    cluster_sync_all();
  }

  __syncthreads();
  if (threadIdx.x == 0) FF_TL(status, KID_GEMM_SKINNY, 11);
  if (bars.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

}  // namespace ff
using namespace ff;

// Pipeline (and cluster receive buffer) bytes a CTA may use: one CTA per SM. FF_SKINNY_SMEM_KB=110 leaves room
// for two, so that under programmatic dependent launch the next kernel's CTAs are resident (barriers, tensor memory,
// first weight stages ready) while this kernel still streams; measured slower (6.82 against 6.13 ms per Llama-3-8B
// decode step at batch 64): the waiting CTAs' polling and early weight requests take more from the running kernel
// than their head start gives back.
static int sk_smem_limit() {
  static int v = 0;
  if (v == 0) {
    v = 200 * 1024;
    if (const char* ev = getenv("FF_SKINNY_SMEM_KB")) { const int kb = atoi(ev); if (kb >= 64 && kb <= 200) v = kb * 1024; }
  }
  return v;
}
constexpr int SK_SMEM_FULL = 200 * 1024;        // budget of a CTA that has its SM to itself (more than 64 tokens)
// budget for a launch of M tokens: the split of a problem is chosen for 64 tokens under the small budget and kept for
// every M (a row's bits must not depend on the batch it is computed in); only the pipeline depth follows M
static int sk_smem_for(int M) { return M <= 64 ? sk_smem_limit() : SK_SMEM_FULL; }

// Largest number of co-resident clusters of `s` CTAs of this kernel (0 when such a cluster cannot be
// launched); queried once per cluster size.
static int skinny_max_clusters(int s) {
  static int cache[FF_MAX_DEVICES][9];
  static bool cache_init = false;
  if (!cache_init) { for (auto& row : cache) for (int& v : row) v = -1; cache_init = true; }
  if (s < 2 || s > 8) return 0;
  int* cached = cache[current_device()];
  if (cached[s] >= 0) return cached[s];
  auto kern = gemm_skinny_kernel<false>;
  if (opt_in_smem(kern, SK_SMEM_FULL + 1024)) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(s * 64); cfg.blockDim = dim3(192); cfg.dynamicSmemBytes = SK_SMEM_FULL + 1024;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = s; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
  cached[s] = n;
  return n;
}

// Decomposition of a problem. cluster == 1: persistent stream-K over tiles of tile_rows weight rows.
// cluster > 1: cluster split-K, one cluster per tile, `tiles` clusters.
struct SkinnyConfig { int cluster, tile_rows, tiles, stages, pipe_off; };

// bytes behind the last stage that the 128-row UMMA read of its activation tile may still touch
static int skinny_tail_slack(int ntok, int tile_rows) {
  const int stage = (ntok + tile_rows) * SBK * 2;
  return stage >= STOK * SBK * 2 ? 0 : STOK * SBK * 2 - stage;
}

static int skinny_stages(int tile_rows, int reserved = 0, int ntok = 64, int limit = 0) {
  if (limit == 0) limit = sk_smem_limit();
  int st = (limit - reserved - skinny_tail_slack(ntok, tile_rows)) / ((ntok + tile_rows) * SBK * 2);
  if (st > SK_MAX_STAGES) st = SK_MAX_STAGES;
  if (const char* ev = getenv("FF_SKINNY_STAGES")) { const int v = atoi(ev); if (v >= 2 && v < st) st = v; }
  return st;
}

// Calibrated decompositions: (N, K, epi) -> (cluster size, tile rows), written by the calibration run (or loaded from
// its cache) and consulted before the time model below. Keyed without M on purpose: a row's bits must not depend on
// the batch it is computed in. The counterpart of the reference's measured linear choices
// (src/backend/cuda/linear_calibrate.rs, src/backend/setup.rs:223-256).
struct SkinnyChoice { int N, K, epi, s, rows; };
static std::mutex g_choice_mu;
static std::vector<SkinnyChoice> g_choices;

static bool skinny_choice(int N, int K, int epi, int* s, int* rows) {
  std::lock_guard<std::mutex> lk(g_choice_mu);
  for (const SkinnyChoice& c : g_choices)
    if (c.N == N && c.K == K && c.epi == epi) { *s = c.s; *rows = c.rows; return true; }
  return false;
}

static void skinny_fit_cluster(SkinnyConfig& c, int M, int N, int epi) {
  const int s = c.cluster, ntok = (M + 15) / 16 * 16;
  while (true) {
    c.pipe_off = (s * ((M + s - 1) / s) * (c.tile_rows + SP_PAD) * 4 + 1023) / 1024 * 1024;
    c.stages = skinny_stages(c.tile_rows, c.pipe_off, ntok, sk_smem_for(M));
    if (c.stages >= 3 || epi != 0 || c.tile_rows <= 64) break;
    c.tile_rows = (c.tile_rows / 2 + 15) / 16 * 16;
    c.tiles = (N + c.tile_rows - 1) / c.tile_rows;
  }
}

// epi != 0 (row-wise epilogue): tiles are exactly 128 rows.
static SkinnyConfig skinny_config(int M, int N, int K, int epi = 0) {
  const int kblocks = (K + SBK - 1) / SBK;
  static int env_s = -1, env_r = -1;
  if (env_s < 0) {
    const char* a = getenv("FF_SKINNY_S"); const char* b = getenv("FF_SKINNY_R");
    env_s = a ? atoi(a) : 0; env_r = b ? atoi(b) : 0;
  }
  // stream-K: widest tile that N fills
  int rows1 = 128;                               // measured: 128-row tiles beat 256 (the fix-up moves half the bytes)
  if (N < rows1) rows1 = (N + 15) / 16 * 16;
  if (env_r > 0 && env_s == 1 && epi == 0) rows1 = env_r;
  SkinnyConfig best = {1, rows1, (N + rows1 - 1) / rows1, skinny_stages(rows1), 0};
  if (env_s == 1) return best;
  int cal_s = 0, cal_r = 0;
  if (env_s <= 0 && skinny_choice(N, K, epi, &cal_s, &cal_r)) {
    if (cal_s == 1) {
      if (epi == 0 && cal_r >= 16 && cal_r <= SBN && cal_r % 16 == 0 && N >= cal_r)
        best = {1, cal_r, (N + cal_r - 1) / cal_r, skinny_stages(cal_r), 0};
      best.stages = skinny_stages(best.tile_rows, 0, (M + 15) / 16 * 16, sk_smem_for(M));
      return best;
    }
    // a cluster choice is taken only while it is launchable here (the table may come from another device)
    const int rows = epi != 0 ? 128 : cal_r;
    const int tiles = rows > 0 ? (N + rows - 1) / rows : 0;
    const int maxc = (cal_s >= 2 && cal_s <= 8) ? skinny_max_clusters(cal_s) - (cal_s > 2 ? 1 : 0) : 0;
    if (rows >= 64 && rows <= SBN && rows % 16 == 0 && kblocks / cal_s >= 2 && tiles <= maxc) {
      const int recv64 = (cal_s * ((64 + cal_s - 1) / cal_s) * (rows + SP_PAD) * 4 + 1023) / 1024 * 1024;
      if (skinny_stages(rows, recv64) >= 3) {
        best = {cal_s, rows, tiles, 0, 0};
        skinny_fit_cluster(best, M, N, epi);
        return best;
      }
    }
  }
  // Time model (microseconds). A CTA takes in at most ~60 GB/s (weights plus the activation tile it
  // re-reads from L2 for every k-block), a pipeline of `st` stages cannot turn a k-block around faster
  // than the ~1.5 us load latency / st, and all CTAs together cannot beat HBM (~5.9 TB/s on reads).
  // The choice must not depend on M: the K split fixes the order of the FP32 additions, and a
  // row's bits may not change with the batch it is computed in. So the model assumes 64 tokens and
  // the receive buffer is sized for those 64 (more tokens get the larger shared-memory budget and the same split).
  const int ntok = 64;
  (void)M;
  auto model = [&](int rows, int kb_per_cta, int st, double ctas) {
    const double per_kb = (rows + ntok) * 128.0 / 60e3;
    const double lat_kb = 1.5 / st;
    const double t_cta = kb_per_cta * (per_kb > lat_kb ? per_kb : lat_kb);
    const double t_hbm = (double)N * K * 2.0 / 5.9e6;
    (void)ctas;
    return t_cta > t_hbm ? t_cta : t_hbm;
  };
  const long long units = (long long)best.tiles * kblocks;
  const int g1 = (int)(units / 2 > 148 ? 148 : (units / 2 < 1 ? 1 : units / 2));
  // stream-K pays a trip through global scratch for the partial tiles: about 4 us on top
  double best_cost = model(rows1, (int)((units + g1 - 1) / g1), best.stages, g1) + (g1 > best.tiles ? 4.0 : 0.0);
  for (int s = 2; s <= 8; ++s) {
    if (env_s > 0 && s != env_s) continue;
    if (kblocks / s < 2) continue;
    // one cluster slot is left free: a launch that needs every slot can find one taken when it starts
    // while the preceding kernel drains (programmatic dependent launch), and then runs in two waves
    const int maxc = skinny_max_clusters(s) - (s > 2 ? 1 : 0);
    if (maxc <= 0) continue;
    for (int rows = 64; rows <= SBN; rows += 16) {
      if (epi != 0 && rows != 128) continue;
      if (epi == 0 && env_r > 0 && rows != env_r) continue;
      const int tiles = (N + rows - 1) / rows;
      if (tiles > maxc) continue;
      // receive buffer: S slots x ceil(M/S) rows of (rows + pad) floats, in front of the pipeline
      const int recv = (s * ((ntok + s - 1) / s) * (rows + SP_PAD) * 4 + 1023) / 1024 * 1024;
      const int st = skinny_stages(rows, recv);
      if (st < 3) continue;
      const double c = model(rows, (kblocks + s - 1) / s, st, (double)tiles * s);
      if (c < best_cost - 1e-9 || (env_s > 0 && best.cluster == 1)) { best_cost = c; best = {s, rows, tiles, st, recv}; }
    }
  }
  if (best.cluster > 1) {
    // the K split (cluster size) is fixed above for every M: it alone decides the order of the FP32 additions of an
    // output element. The receive buffer and with it the pipeline depth follow the actual M; where many tokens and a
    // wide tile leave fewer than three stages, the tile is narrowed (more clusters, possibly a second wave; the bits
    // of every output stay the same)
    skinny_fit_cluster(best, M, N, epi);
  } else {
    best.stages = skinny_stages(best.tile_rows, 0, (M + 15) / 16 * 16, sk_smem_for(M));
  }
  return best;
}

// Decomposition chosen for a problem: out = {cluster size, tile rows, tiles, pipeline stages, grid}.
FF_EXPORT int ff_gemm_skinny_config(int M, int N, int K, int epi, int* out) {
  if (M <= 0 || M > STOK || N <= 0 || K <= 0 || out == nullptr) return FF_HOST_BAD_SHAPE;
  const SkinnyConfig c = skinny_config(M, N, K, epi);
  long long sb = 0, cb = 0;
  out[0] = c.cluster; out[1] = c.tile_rows; out[2] = c.tiles; out[3] = c.stages;
  out[4] = (c.cluster > 1) ? c.tiles * c.cluster : 0;
  (void)sb; (void)cb;
  return 0;
}

// Record (s >= 1) or forget (s == 0) the calibrated decomposition of every decode GEMM with this (N, K, epi):
// s = 1 stream-K with `rows`-row tiles, s = 2..8 cluster split-K. A choice that is not launchable is ignored at plan time.
FF_EXPORT int ff_gemm_skinny_set_choice(int N, int K, int epi, int s, int rows) {
  if (N <= 0 || K <= 0 || s < 0 || s > 8) return FF_HOST_BAD_SHAPE;
  std::lock_guard<std::mutex> lk(g_choice_mu);
  for (size_t i = 0; i < g_choices.size(); ++i)
    if (g_choices[i].N == N && g_choices[i].K == K && g_choices[i].epi == epi) { g_choices.erase(g_choices.begin() + i); break; }
  if (s > 0) g_choices.push_back({N, K, epi, s, rows});
  return 0;
}

// Number of co-resident clusters of `s` CTAs of the decode GEMM on the current device (0: not launchable).
FF_EXPORT int ff_gemm_skinny_max_clusters(int s) { return skinny_max_clusters(s); }

// Plan for a problem: returns the grid size (cluster split-K: tiles x cluster size; otherwise one
// persistent CTA per SM, fewer for tiny problems);
// *scratch_bytes = FP32 partial slots (two per CTA; none in cluster mode), *counter_bytes = one int32
// per weight tile (zero before the first launch; every launch leaves them zero).
static int skinny_plan(int M, int N, int K, int epi, long long* scratch_bytes, long long* counter_bytes) {
  const int kblocks = (K + SBK - 1) / SBK;
  const SkinnyConfig cfg = skinny_config(M, N, K, epi);
  if (counter_bytes) *counter_bytes = (long long)cfg.tiles * 4;
  if (cfg.cluster > 1) {
    if (scratch_bytes) *scratch_bytes = 0;
    return cfg.tiles * cfg.cluster;
  }
  const long long total = (long long)cfg.tiles * kblocks;
  long long g = total / 2;                 // at least two k-blocks of work per CTA
  if (g > 148) g = 148;
  if (g < 1) g = 1;
  if (scratch_bytes) *scratch_bytes = g > 1 ? 2 * g * (long long)M * cfg.tile_rows * 4 : 0;
  return (int)g;
}

FF_EXPORT int ff_gemm_skinny_plan(int M, int N, int K, long long* scratch_bytes, long long* counter_bytes) {
  return skinny_plan(M, N, K, 0, scratch_bytes, counter_bytes);
}

// Plan for the variants with a row-wise epilogue (epi 1 SwiGLU, 2 rotary + KV write): N % 128 == 0.
FF_EXPORT int ff_gemm_skinny_plan_epi(int M, int N, int K, int epi, long long* scratch_bytes, long long* counter_bytes) {
  if (N % 128) return FF_HOST_BAD_SHAPE;
  return skinny_plan(M, N, K, epi, scratch_bytes, counter_bytes);
}

static int gemm_skinny_launch(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                              int grid, float* scratch, int* counters, int* status, cudaStream_t stream,
                              const PeerArena* arena, const SkinnyEpi* epi = nullptr) {
  if (M <= 0 || N <= 0 || K <= 0) return FF_HOST_BAD_SHAPE;
  SkinnyEpi ep = {};
  if (epi != nullptr) {
    ep = *epi;
    if (arena != nullptr || (N % 128) || (ldy % 8) || (reinterpret_cast<uintptr_t>(Y) & 15)) return FF_HOST_BAD_SHAPE;
  }
  if (M > STOK) return FF_HOST_TOO_LARGE;
  if ((K % 8) || (ldx % 8) || (ldw % 8)) return FF_HOST_BAD_ALIGN;
  const SkinnyConfig cfg = skinny_config(M, N, K, ep.mode);
  const int cl = cfg.cluster;
  const long long total = (long long)cfg.tiles * ((K + SBK - 1) / SBK);
  if (cl > 1) {
    if (grid != cfg.tiles * cl) return FF_HOST_BAD_SHAPE;
    if (arena != nullptr && cfg.tiles * cl > MAX_FLAGS / 2) return FF_HOST_TOO_LARGE;
  } else {
    if (grid < 1 || grid > 1024 || (grid > 1 && (scratch == nullptr || counters == nullptr))) return FF_HOST_BAD_SHAPE;
    if (grid > total) return FF_HOST_BAD_SHAPE;
    if (arena != nullptr && cfg.tiles > MAX_FLAGS / 2) return FF_HOST_TOO_LARGE;
  }
  const int ntok = (M + 15) / 16 * 16;
  CUtensorMap tmX, tmW;
  int r = make_tmap_2d(&tmX, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, (uint64_t)ldx * 2, SBK, ntok);
  if (r) return r;
  r = make_tmap_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, (uint64_t)ldw * 2, SBK, cfg.tile_rows);
  if (r) return r;
  if (cfg.stages < 2) return FF_HOST_TOO_LARGE;
  const int smem = cfg.pipe_off + cfg.stages * (ntok + cfg.tile_rows) * SBK * 2 + skinny_tail_slack(ntok, cfg.tile_rows) + 1024;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(Y);
  if (arena == nullptr) {
    auto kern = gemm_skinny_kernel<false>;
    r = opt_in_smem(kern, SK_SMEM_FULL + 1024); if (r) return r;
    PeerArena none = {};
    return launch_pdl(kern, dim3(grid), dim3(192), smem, stream, cl, tmX, tmW, y, M, N, K, ldy, ntok, cfg.tile_rows,
                      cfg.stages, cl, cfg.pipe_off, scratch, counters, status, none, ep);
  }
  auto kern = gemm_skinny_kernel<true>;
  r = opt_in_smem(kern, SK_SMEM_FULL + 1024); if (r) return r;
  return launch_pdl(kern, dim3(grid), dim3(192), smem, stream, cl, tmX, tmW, y, M, N, K, ldy, ntok, cfg.tile_rows,
                    cfg.stages, cl, cfg.pipe_off, scratch, counters, status, *arena, ep);
}

// `grid` is the value returned by ff_gemm_skinny_plan for the same problem.
FF_EXPORT int ff_gemm_skinny(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                             int grid, float* scratch, int* counters, int* status, cudaStream_t stream) {
  return gemm_skinny_launch(X, W, Y, M, N, K, ldx, ldw, ldy, grid, scratch, counters, status, stream, nullptr);
}

// Gate/up projection with the SwiGLU applied in the epilogue: W is [N, K] with gate/up rows interleaved per
// 64, Y is [M, N/2]. `grid` from ff_gemm_skinny_plan_epi(M, N, K, 1).
FF_EXPORT int ff_gemm_skinny_swiglu(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                                    int grid, float* scratch, int* counters, int* status, cudaStream_t stream) {
  SkinnyEpi ep = {};
  ep.mode = 1;
  return gemm_skinny_launch(X, W, Y, M, N, K, ldx, ldw, ldy, grid, scratch, counters, status, stream, nullptr, &ep);
}

// Fused QKV projection with rotary embedding and paged KV-cache write in the epilogue (128-dim heads;
// N = (hq + 2*hkv) * 128). Y receives the rotated Q/K and V rows; K and V also go to `slots` of the cache
// (layout [blocks, hkv, block_size, 128]; negative slots are skipped). cos_sin: [M, rot_dim/2] float pairs from
// ff_rope_table. `grid` from
// ff_gemm_skinny_plan_epi(M, N, K, 2).
FF_EXPORT int ff_gemm_skinny_rope_kv(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                                     int grid, float* scratch, int* counters, const float* cos_sin, const int* slots,
                                     void* kcache, void* vcache, int hq, int hkv, int rot_dim, int block_size,
                                     int num_blocks, int* status, cudaStream_t stream) {
  if (hq <= 0 || hkv <= 0 || N != (hq + 2 * hkv) * 128 || rot_dim > 128 || rot_dim % 2) return FF_HOST_BAD_SHAPE;
  SkinnyEpi ep = {};
  ep.mode = 2; ep.cos_sin = reinterpret_cast<const float2*>(cos_sin); ep.slots = slots;
  ep.kcache = static_cast<__nv_bfloat16*>(kcache); ep.vcache = static_cast<__nv_bfloat16*>(vcache);
  ep.hq = hq; ep.hkv = hkv; ep.rot_dim = rot_dim; ep.block_size = block_size; ep.num_blocks = num_blocks;
  return gemm_skinny_launch(X, W, Y, M, N, K, ldx, ldw, ldy, grid, scratch, counters, status, stream, nullptr, &ep);
}

// Row-parallel projection fused with the tensor-parallel all-reduce (decode shapes, M <= 128):
// Y = sum over ranks of X_r · W_rᵀ, identical bits on every rank. ptrs: arena base of every rank.
FF_EXPORT int ff_gemm_ar(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                         long long slot_bytes, const void* X, const void* W, void* Y, int M, int N, int K, int ldx,
                         int ldw, int ldy, int grid, float* scratch, int* counters, unsigned long long mc_ptr, int* status,
                         cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return FF_HOST_BAD_SHAPE;
  if (N % 8 || (long long)M * N * 2 > slot_bytes || half_bytes < slot_bytes * world) return FF_HOST_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(Y) & 15) || (ldy % 8) || (slot_bytes % 16)) return FF_HOST_BAD_ALIGN;
  PeerArena a = {};
  for (int i = 0; i < MAX_RANKS; ++i) a.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  a.rank = rank; a.world = world; a.half_bytes = half_bytes; a.slot_bytes = slot_bytes;
  // mc_ptr != 0: the arena's NVLS multicast mapping; the exchange then goes through the switch (two-shot)
  a.mc_base = reinterpret_cast<uint8_t*>(mc_ptr);
  if (mc_ptr != 0 && world < 2) a.mc_base = nullptr;
  // one-shot (default): every rank multicasts its partial (multimem.st) and one flag, then sums all slots locally: one
  // flag round instead of the two of the reduce-in-the-switch exchange (FF_NVLS_ONESHOT=0 selects that one)
  static const int oneshot = [] { const char* ev = getenv("FF_NVLS_ONESHOT"); return (ev && ev[0] == '0') ? 0 : 1; }();
  a.mc_oneshot = a.mc_base != nullptr ? oneshot : 0;
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
//  * Limit: the partial-sum slots (2 * grid * M * 128 * 4 bytes for a problem that runs as stream-K over
//    128-row weight tiles, grid <= 148 persistent CTAs; none when the problem runs as cluster
//    split-K) must fit in FF_NOALLOC_SCRATCH_BYTES (8 MiB) and the weight tiles in
//    FF_NOALLOC_MAX_TILES (2048); larger problems are refused with FF_HOST_TOO_LARGE (for wide layers
//    that fill all 148 CTAs this means M <= 55 tokens), and so is M > 128.
//    Every GPU that loads this library holds the 8 MiB until exit.
//  * The first call on a device resolves the device addresses of the arrays
//    (cudaGetSymbolAddress, with that device current) and caches them; make that first call
//    before starting any stream capture. The current device must be the one `stream` belongs to.
//    The per-device cache is guarded by a mutex, so first calls may come from several host threads.
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
static NoAllocPtrs g_noalloc_ptrs[FF_MAX_DEVICES] = {};
static std::mutex g_noalloc_mu;
}  // namespace ff

FF_EXPORT int ff_gemm_skinny_noalloc(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                     int ldy, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return FF_HOST_BAD_SHAPE;
  if (M > STOK) return FF_HOST_TOO_LARGE;
  long long scratch_bytes = 0, counter_bytes = 0;
  const int grid = ff_gemm_skinny_plan(M, N, K, &scratch_bytes, &counter_bytes);
  if (scratch_bytes > (long long)FF_NOALLOC_SCRATCH_BYTES || counter_bytes > (long long)FF_NOALLOC_MAX_TILES * 4)
    return FF_HOST_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= FF_MAX_DEVICES) return FF_HOST_UNSUPPORTED;
  NoAllocPtrs p;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    NoAllocPtrs& slot = g_noalloc_ptrs[dev];
    if (!slot.ready) {
      // In host code the array names are host-side stand-ins; the kernel needs the device address.
      void* ps = nullptr; void* pc = nullptr;
      e = cudaGetSymbolAddress(&ps, g_noalloc_scratch);
      if (e != cudaSuccess) return static_cast<int>(e);
      e = cudaGetSymbolAddress(&pc, g_noalloc_counters);
      if (e != cudaSuccess) return static_cast<int>(e);
      slot.scratch = static_cast<float*>(ps); slot.counters = static_cast<int*>(pc); slot.ready = true;
    }
    p = slot;
  }
  e = cudaMemsetAsync(p.counters, 0, (size_t)counter_bytes, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  return ff_gemm_skinny(X, W, Y, M, N, K, ldx, ldw, ldy, grid, p.scratch, p.counters, status, stream);
}
