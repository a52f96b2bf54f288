// BF16 linear layers on 5th-generation tensor cores:  Y[M,N] = X[M,K] · W[N,K]ᵀ
// (activations row-major, weights in the checkpoint's [out, in] layout, FP32 accumulation,
// one BF16 rounding at the end).
//
// gemm_bf16_kernel serves M > 128 (prefill, verification batches): a warp-specialised pipeline
// (TMA producer warp -> mbarrier ring -> single-thread tcgen05.mma issuer -> TMEM accumulator ->
// 4 epilogue warps), persistent over 128 x BN x 64 tiles with double-buffered TMEM accumulators so
// the epilogue of tile i overlaps the mainloop of tile i+1. Optional fused SwiGLU epilogue
// (gate|up interleaved per 64 rows of the weight), grouped mode for expert segments, and the
// tensor-parallel forms (all-gather -> GEMM, GEMM -> reduce-scatter) with peer stores in the same
// kernel. Decode shapes (M <= 128) are served by gemm_skinny.cu.
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

// Grouped mode (mixture-of-experts prefill): the rows of A are expert segments (segment e starts at row
// seg_off[e], a multiple of 16, and holds counts[e] rows), B stacks the experts' weights (expert e at row
// e * N). Segment e contributes ceil(counts[e] / 128) row tiles x tiles_n column tiles, row tile fastest,
// so the CTAs working side by side share one weight tile and the segment's rows stay in L2. A row tile may
// reach past its segment: those rows are computed and not stored.
struct GroupArgs {
  const int* seg_off;                 // nullptr: dense problem
  const int* counts;
  int E;
};

struct TileWalk { int e = 0, base = 0; };

// Operand rows of linear tile t of this CTA's loop (t grows monotonically); false when the problem is done.
__device__ __forceinline__ bool next_tile(const GroupArgs& g, TileWalk& w, int t, int tiles_m, int tiles_n,
                                          int M, int N, int BN, int& tm, int& tn, int& a_row0, int& b_row0,
                                          int& row_end) {
  if (g.seg_off == nullptr) {
    if (t >= tiles_m * tiles_n) return false;
    tile_coords(t, tiles_m, tiles_n, tm, tn);
    a_row0 = tm * BM; b_row0 = tn * BN; row_end = M;
    return true;
  }
  while (w.e < g.E) {
    // a segment reaching past the row buffers (an overflowed dispatch, reported through the status word) is cut there
    const int cnt = max(0, min(g.counts[w.e], M - g.seg_off[w.e]));
    const int tme = (cnt + BM - 1) / BM;
    const int n = tme * tiles_n;
    if (t < w.base + n) {
      const int tl = t - w.base;
      tm = tl % tme; tn = tl / tme;
      a_row0 = g.seg_off[w.e] + tm * BM;
      b_row0 = w.e * N + tn * BN;
      row_end = g.seg_off[w.e] + cnt;
      return true;
    }
    w.base += n; ++w.e;
  }
  return false;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// epi: 0 = store bf16; 1 = SwiGLU (every 128 columns of a tile are 64 gate then the matching 64 up columns; output
// has N/2 columns); 2 = store fp32.
// COMM (tensor-parallel prefill, rows split evenly over the ranks in 128-row blocks):
//   1 = all-gather -> GEMM : A is row-sharded. Four extra warps per CTA (all CTAs together) push this
//       rank's shard into every peer's arena with plain peer stores, a quarter of a 128-row block at a
//       time, eight 16-byte vectors in flight per thread; the CTA that completes a block (counter)
//       flags it on every peer. The TMA producer reads own rows straight from the shard and the other
//       ranks' rows from the LOCAL arena copy once the block's flag is there; own rows are scheduled
//       first so the transfer overlaps the math.
//   2 = GEMM -> reduce-scatter : every finished tile goes into the arena slot of the rank that owns
//       those rows. The epilogue stages 64 columns at a time through shared memory and every lane hands
//       its row to the copy engine as one 128-byte bulk store (cp.async.bulk shared -> peer global).
//       When all column tiles of a row block are out, its flag goes to the owner.
//       After its tiles every CTA reduces quarter row blocks this rank owns: waits for the block's
//       flags from all ranks and sums the slots in rank order.
struct CommArgs {
  PeerArena ar;
  int rows_per_rank;                  // multiple of 128; M == rows_per_rank * world
  int* tile_counters;                 // COMM 2: int32 per row tile, zero before the first launch
  __nv_bfloat16* rs_out;              // COMM 2: [rows_per_rank, N]
  const __nv_bfloat16* x_shard;       // COMM 1: [rows_per_rank, K]
  int ldx;
};

template <int COMM>
__device__ __forceinline__ int comm_tm(int tm, int tiles_per_rank, int rank, int world) {
  if (COMM != 1) return tm;
  // logical order: own rows first, then the ranks after me
  const int j = tm / tiles_per_rank, r = tm - j * tiles_per_rank;
  return ((rank + j) % world) * tiles_per_rank + r;
}

constexpr int RS_STG_PITCH = 144, RS_STG_BYTES = 32 * RS_STG_PITCH;   // COMM 2 epilogue staging, per warp
constexpr int COMM_PARTS = 4;       // a 128-row block is pushed (COMM 1) / reduced (COMM 2) in this many pieces

template <int BN, int STAGES, int COMM>
__global__ void __launch_bounds__(COMM == 1 ? 320 : 192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmA1,
                 const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmB, void* __restrict__ Cout, int M, int N, int K, int ldc, int epi,
                 int* status, CommArgs ca, GroupArgs ga) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ PipeBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int A_BYTES = BM * BK * 2;
  constexpr int B_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;   // 256 or 512, power of two
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int kblocks = (K + BK - 1) / BK;
  const int tiles_per_rank = COMM ? ca.rows_per_rank / BM : 1;
  int epoch = 0;
  if (COMM) epoch = ld_volatile(arena_epoch(ca.ar)) + 1;
  const int parity = epoch & 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.tmem_full[i], 1); mbar_init(&bars.tmem_empty[i], 4); }
    bars.abort_flag = 0; bars.is_last = 0;
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
      TileWalk walk;
      for (int t = blockIdx.x; ok; t += gridDim.x) {
        int tm, tn, a_row0, b_row0, row_end;
        if (!next_tile(ga, walk, t, tiles_m, tiles_n, M, N, BN, tm, tn, a_row0, b_row0, row_end)) break;
        if (COMM) { tm = comm_tm<COMM>(tm, tiles_per_rank, ca.ar.rank, ca.ar.world); a_row0 = tm * BM; }
        const int src = tm / tiles_per_rank, rb = tm - src * tiles_per_rank;
        if (COMM == 1 && src != ca.ar.rank) {
          // the rows of this tile must have arrived in the local arena copy
          if (!wait_flag(arena_flag(ca.ar, ca.ar.rank, src, rb), epoch, status, KID_AG_GEMM, src)) {
            bars.abort_flag = 1; ok = false; break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");     // peer-written data -> visible to the TMA engine
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES; const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_GEMM_BF16, 1)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], STAGE_BYTES);
          uint8_t* sa = smem + s * STAGE_BYTES;
          if (COMM == 1 && src == ca.ar.rank) tma_load_2d(sa, &tmX, &bars.full[s], kb * BK, rb * BM);
          else if (COMM == 1) tma_load_3d(sa, parity ? &tmA1 : &tmA, &bars.full[s], kb * BK, rb * BM, src);
          else tma_load_2d(sa, &tmA, &bars.full[s], kb * BK, a_row0);
          tma_load_2d(sa + A_BYTES, &tmB, &bars.full[s], kb * BK, b_row0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(1, 1, 0, 0, BM, BN);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      TileWalk walk;
      for (int t = blockIdx.x; ok; t += gridDim.x, ++tile_it) {
        int tm_, tn_, a_, b_, re_;
        if (!next_tile(ga, walk, t, tiles_m, tiles_n, M, N, BN, tm_, tn_, a_, b_, re_)) break;
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
  } else if (warp < 6) {
    // epilogue warps 2..5 ; TMEM lane quarter = warp % 4
    const int q = warp & 3;
    const int e = (warp - 2) * 32 + lane;
    uint32_t tile_it = 0;
    bool ok = true;
    TileWalk walk;
    for (int t = blockIdx.x; ok; t += gridDim.x, ++tile_it) {
      int tm, tn, a_row0, b_row0, row_end;
      if (!next_tile(ga, walk, t, tiles_m, tiles_n, M, N, BN, tm, tn, a_row0, b_row0, row_end)) break;
      if (COMM) { tm = comm_tm<COMM>(tm, tiles_per_rank, ca.ar.rank, ca.ar.world); a_row0 = tm * BM; }
      const int acc = tile_it & 1; const uint32_t aph = (tile_it >> 1) & 1;
      if (!mbar_wait(&bars.tmem_full[acc], aph, abort_flag, status, KID_GEMM_BF16, 4)) { ok = false; break; }
      tc_fence_after();
      const int row = a_row0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      if (epi == 1) {
        constexpr int HALF = BN / 2;
        __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(Cout) + (size_t)row * ldc + (size_t)tn * HALF;
        const int ncols_out = N / 2;
#pragma unroll 1
        for (int c = 0; c < HALF; c += 16) {
          uint32_t g[16], u[16];
          const int gc = (c >> 6) * 128 + (c & 63);      // 64 gate columns, then the matching 64 up columns
          tmem_ld_x16(taddr + gc, g);
          tmem_ld_x16(taddr + gc + 64, u);
          tmem_ld_wait();
          if (row < row_end) {
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
          if (row < row_end) {
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
        if (COMM == 2) {
          // the rows of this tile belong to rank `owner`: they go into its arena slot for source = me,
          // 64 columns at a time through a warp-private staging tile
          const int owner = tm / tiles_per_rank;
          __nv_bfloat16* tile_dst = reinterpret_cast<__nv_bfloat16*>(arena_slot(ca.ar, owner, parity, ca.ar.rank)) +
                                    (size_t)(tm * BM + q * 32 - owner * ca.rows_per_rank) * N + (size_t)tn * BN;
          // staging: lane = row, 64 columns (128 bytes) per pass at a 144-byte pitch (16-byte stores of the 32
          // lanes then fall into distinct bank groups). Each lane hands its own row to the copy engine as one
          // 128-byte bulk store; the staging row is reused as soon as the engine has READ it.
          uint8_t* stg = smem + STAGES * STAGE_BYTES + q * RS_STG_BYTES + lane * RS_STG_PITCH;
          const bool row_ok = tm * BM + q * 32 + lane < M;
#pragma unroll 1
          for (int c = 0; c < BN; c += 64) {
            if (c) tma_store_wait_read<0>();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t r[32];
              tmem_ld_x32(taddr + c + 32 * h, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 4; ++j)
                reinterpret_cast<uint4*>(stg)[4 * h + j] =
                    make_uint4(pack_bf16x2(__uint_as_float(r[8 * j + 0]), __uint_as_float(r[8 * j + 1])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5])),
                               pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7])));
            }
            fence_proxy_async_smem();
            const int col = tn * BN + c;
            if (row_ok && col + 64 <= N) {
              bulk_store(tile_dst + (size_t)lane * N + c, stg, 128);
            } else if (row_ok) {
              for (int ch = 0; ch < 8; ++ch)
                if (col + ch * 8 < N)
                  *reinterpret_cast<uint4*>(tile_dst + (size_t)lane * N + c + ch * 8) = reinterpret_cast<uint4*>(stg)[ch];
            }
            tma_store_commit();
          }
          tma_store_wait<0>();                              // every row of this tile has landed in the owner's slot
          asm volatile("fence.proxy.async;" ::: "memory");
        } else
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_x32(taddr + c, r);
          tmem_ld_wait();
          if (row < row_end) {
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
      if (COMM == 2) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e == 0) {
          __threadfence_system();
          const int prev = atomicAdd(&ca.tile_counters[tm], 1);
          if (prev == tiles_n - 1) {                      // last column tile of this row block on this rank
            ca.tile_counters[tm] = 0;
            __threadfence_system();
            const int owner = tm / tiles_per_rank;
            st_release_sys(arena_flag(ca.ar, owner, ca.ar.rank, tm - owner * tiles_per_rank), epoch);
          }
        }
      }
    }
    if (COMM == 2 && ok) {
      // reduce the row blocks this rank owns, a quarter block per step and CTA: slots of all source
      // ranks, in rank order, sixteen 16-byte vectors in flight per thread
      const int nvec = N >> 3;
      const int blk_vecs = BM * nvec, piece = (blk_vecs + COMM_PARTS - 1) / COMM_PARTS;
      for (int part = blockIdx.x; part < tiles_per_rank * COMM_PARTS; part += gridDim.x) {
        const int i = part / COMM_PARTS, ps = part - i * COMM_PARTS;
        if (e == 0) bars.is_last = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (e < ca.ar.world)
          if (!wait_flag(arena_flag(ca.ar, ca.ar.rank, e, i), epoch, status, KID_GEMM_RS, e)) bars.is_last = 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (bars.is_last) {
          const int v0 = ps * piece, v1 = min(blk_vecs, v0 + piece);
          // eight vectors per thread and slot, the next slot's loads issued before the current one is summed:
          // with one CTA per SM the reduction is bound by loads in flight, not by bandwidth
          constexpr int U = 8;
          for (int base = v0 + e; base < v1; base += 128 * U) {
            float a8[U][8];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
              for (int j = 0; j < 8; ++j) a8[u][j] = 0.f;
            uint4 cur[U], nxt[U];
            const uint4* slot0 = reinterpret_cast<const uint4*>(arena_slot(ca.ar, ca.ar.rank, parity, 0)) + (size_t)i * blk_vecs;
#pragma unroll
            for (int u = 0; u < U; ++u) cur[u] = (base + 128 * u < v1) ? __ldcg(slot0 + base + 128 * u) : make_uint4(0, 0, 0, 0);
            for (int r = 0; r < ca.ar.world; ++r) {
              if (r + 1 < ca.ar.world) {
                const uint4* slot = reinterpret_cast<const uint4*>(arena_slot(ca.ar, ca.ar.rank, parity, r + 1)) + (size_t)i * blk_vecs;
#pragma unroll
                for (int u = 0; u < U; ++u) nxt[u] = (base + 128 * u < v1) ? __ldcg(slot + base + 128 * u) : make_uint4(0, 0, 0, 0);
              }
#pragma unroll
              for (int u = 0; u < U; ++u) {
                const uint32_t* dp = reinterpret_cast<const uint32_t*>(&cur[u]);
#pragma unroll
                for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(dp[j]); a8[u][2 * j] += f.x; a8[u][2 * j + 1] += f.y; }
              }
#pragma unroll
              for (int u = 0; u < U; ++u) cur[u] = nxt[u];
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (base + 128 * u < v1) {
                uint4 o;
                o.x = pack_bf16x2(a8[u][0], a8[u][1]); o.y = pack_bf16x2(a8[u][2], a8[u][3]);
                o.z = pack_bf16x2(a8[u][4], a8[u][5]); o.w = pack_bf16x2(a8[u][6], a8[u][7]);
                reinterpret_cast<uint4*>(ca.rs_out)[(size_t)i * blk_vecs + base + 128 * u] = o;
              }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
    }
    if (COMM && e == 0) {
      __threadfence();
      const int prev = atomicAdd(arena_done(ca.ar), 1);
      if (prev == (int)gridDim.x - 1) {
        *arena_done(ca.ar) = 0;
        __threadfence();
        *reinterpret_cast<volatile int*>(arena_epoch(ca.ar)) = epoch;
      }
    }
  }

  if (COMM == 1 && warp >= 6) {
    // ---- communication warps 6..9: push this rank's shard to every peer --------------------------
    const int ce = threadIdx.x - 192;                    // 0..127
    const int kvec = K >> 3;
    const int blk_vecs = BM * kvec, piece = (blk_vecs + COMM_PARTS - 1) / COMM_PARTS;
    for (int part = blockIdx.x; part < tiles_per_rank * COMM_PARTS; part += gridDim.x) {
      const int rb = part / COMM_PARTS, ps = part - rb * COMM_PARTS;
      const int v0 = ps * piece, v1 = min(blk_vecs, v0 + piece);
      for (int pi = 1; pi < ca.ar.world; ++pi) {
        const int p = (ca.ar.rank + pi) % ca.ar.world;
        uint4* dst = reinterpret_cast<uint4*>(arena_slot(ca.ar, p, parity, ca.ar.rank)) + (size_t)rb * blk_vecs;
        for (int base = v0 + ce; base < v1; base += 128 * 8) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int idx = base + 128 * j;
            if (idx < v1) {
              const int r = idx / kvec, c = idx - r * kvec;
              v[j] = reinterpret_cast<const uint4*>(ca.x_shard + (size_t)(rb * BM + r) * ca.ldx)[c];
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) if (base + 128 * j < v1) dst[base + 128 * j] = v[j];
        }
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ce == 0) {
        __threadfence_system();
        const int prev = atomicAdd(&ca.tile_counters[rb], 1);
        if (prev == COMM_PARTS - 1) {                      // the last piece of this row block is out
          ca.tile_counters[rb] = 0;
          __threadfence_system();
          for (int pi = 1; pi < ca.ar.world; ++pi)
            st_release_sys(arena_flag(ca.ar, (ca.ar.rank + pi) % ca.ar.world, ca.ar.rank, rb), epoch);
        }
      }
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
  auto kern = gemm_bf16_kernel<BN, STAGES, 0>;
  r = opt_in_smem(kern, smem); if (r) return r;
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  CommArgs none = {};
  kern<<<grid, 192, smem, stream>>>(tmA, tmA, tmA, tmB, Y, M, N, K, ldy, epi, status, none, GroupArgs{});
  return launch_result();
}

// Grouped GEMM over expert segments with 128-row token tiles (prefill sizes; the swap-AB kernel of moe.cu serves
// segments of a few rows): Y[seg rows, Nw] = Xs[seg rows, K] · W[e][Nw, K]ᵀ. Xs [capacity, K] and Y rows are
// addressed by seg_off / counts (device arrays, no host read-back); W is [E_local * Nw, K]. epi 0 / 1 as above.
FF_EXPORT int ff_moe_grouped_gemm_tiled(const void* Xs, const void* W, void* Y, const int* seg_off, const int* counts,
                                        int E_local, int Nw, int K, int capacity, int ldy, int epi, int* status,
                                        cudaStream_t stream) {
  if (E_local <= 0 || Nw <= 0 || K <= 0 || capacity <= 0 || !seg_off || !counts) return FF_HOST_BAD_SHAPE;
  if ((K % 8) || (epi != 0 && epi != 1) || (epi == 1 && (Nw % 256))) return FF_HOST_BAD_SHAPE;
  const int out_cols = (epi == 1) ? Nw / 2 : Nw;
  if (((size_t)ldy * 2) % 16 || ldy < out_cols || (reinterpret_cast<uintptr_t>(Y) & 15)) return FF_HOST_BAD_ALIGN;
  CUtensorMap tmA, tmB;
  constexpr int BN = 256, STAGES = 4;
  int r = make_tmap_2d(&tmA, Xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, capacity, (uint64_t)K * 2, BK, BM);
  if (r) return r;
  r = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, (uint64_t)E_local * Nw, (uint64_t)K * 2, BK, BN);
  if (r) return r;
  const int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto kern = gemm_bf16_kernel<BN, STAGES, 0>;
  r = opt_in_smem(kern, smem); if (r) return r;
  CommArgs none = {};
  GroupArgs ga = {seg_off, counts, E_local};
  kern<<<sm_count(), 192, smem, stream>>>(tmA, tmA, tmA, tmB, Y, capacity, Nw, K, ldy, epi, status, none, ga);
  return launch_result();
}

static int fill_comm(CommArgs& ca, const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                     long long slot_bytes, int M, long long need_slot_bytes) {
  if (world < 2 || world > MAX_RANKS || rank < 0 || rank >= world) return FF_HOST_BAD_SHAPE;
  if (M % (world * BM)) return FF_HOST_BAD_SHAPE;
  if (need_slot_bytes > slot_bytes || half_bytes < slot_bytes * world) return FF_HOST_TOO_LARGE;
  if (M / world / BM > MAX_FLAGS) return FF_HOST_TOO_LARGE;
  for (int i = 0; i < MAX_RANKS; ++i) ca.ar.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  ca.ar.rank = rank; ca.ar.world = world; ca.ar.half_bytes = half_bytes; ca.ar.slot_bytes = slot_bytes;
  ca.rows_per_rank = M / world;
  return 0;
}

// Column-parallel projection fused with the all-gather of its row-sharded input:
// Y[M, N] = gather(X_shards)[M, K] · W[N, K]ᵀ, X_shard = this rank's rows [M/world, K].
FF_EXPORT int ff_ag_gemm(const unsigned long long* ptrs, int rank, int world, long long half_bytes, long long slot_bytes,
                         const void* x_shard, const void* W, void* Y, int M, int N, int K, int ldx, int ldw, int ldy,
                         int epi, int* block_counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8)) return FF_HOST_BAD_SHAPE;
  if (epi == 1 && (N % 256)) return FF_HOST_BAD_SHAPE;
  if (epi == 2) return FF_HOST_UNSUPPORTED;
  const int out_cols = (epi == 1) ? N / 2 : N;
  if ((ldy % 8) || ldy < out_cols || (reinterpret_cast<uintptr_t>(Y) & 15)) return FF_HOST_BAD_ALIGN;
  CommArgs ca = {};
  int r = fill_comm(ca, ptrs, rank, world, half_bytes, slot_bytes, M, (long long)(M / world) * K * 2);
  if (r) return r;
  if (!block_counters) return FF_HOST_BAD_SHAPE;
  ca.x_shard = reinterpret_cast<const __nv_bfloat16*>(x_shard); ca.ldx = ldx;
  ca.tile_counters = block_counters;          // one int32 per 128-row block of the shard, zero between launches
  constexpr int BN = 256, STAGES = 4;
  CUtensorMap tmA0, tmA1, tmX, tmB;
  r = make_tmap_2d(&tmX, x_shard, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, ca.rows_per_rank, (uint64_t)ldx * 2, BK, BM);
  if (r) return r;
  uint8_t* data = reinterpret_cast<uint8_t*>(ptrs[rank]) + DATA_OFF;
  r = make_tmap_3d(&tmA0, data, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, ca.rows_per_rank, world, (uint64_t)K * 2,
                   (uint64_t)slot_bytes, BK, BM, 1);
  if (r) return r;
  r = make_tmap_3d(&tmA1, data + half_bytes, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, ca.rows_per_rank, world,
                   (uint64_t)K * 2, (uint64_t)slot_bytes, BK, BM, 1);
  if (r) return r;
  r = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, (uint64_t)ldw * 2, BK, BN);
  if (r) return r;
  const int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 1024;
  auto kern = gemm_bf16_kernel<BN, STAGES, 1>;
  r = opt_in_smem(kern, smem); if (r) return r;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 320, smem, stream>>>(tmA0, tmA1, tmX, tmB, Y, M, N, K, ldy, epi, status, ca, GroupArgs{});
  return launch_result();
}

// Row-parallel projection fused with the reduce-scatter of its output:
// out[M/world, N] = rows owned by this rank of sum_r X_r[M, K_r] · W_r[N, K_r]ᵀ.
FF_EXPORT int ff_gemm_rs(const unsigned long long* ptrs, int rank, int world, long long half_bytes, long long slot_bytes,
                         const void* X, const void* W, void* out, int M, int N, int K, int ldx, int ldw,
                         int* tile_counters, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || (N % 8)) return FF_HOST_BAD_SHAPE;
  if (!tile_counters || (reinterpret_cast<uintptr_t>(out) & 15)) return FF_HOST_BAD_ALIGN;
  CommArgs ca = {};
  int r = fill_comm(ca, ptrs, rank, world, half_bytes, slot_bytes, M, (long long)(M / world) * N * 2);
  if (r) return r;
  ca.tile_counters = tile_counters; ca.rs_out = reinterpret_cast<__nv_bfloat16*>(out);
  constexpr int BN = 256, STAGES = 4;
  CUtensorMap tmA, tmB;
  r = make_tmap_2d(&tmA, X, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, M, (uint64_t)ldx * 2, BK, BM);
  if (r) return r;
  r = make_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, N, (uint64_t)ldw * 2, BK, BN);
  if (r) return r;
  const int smem = STAGES * (BM * BK * 2 + BN * BK * 2) + 4 * RS_STG_BYTES + 1024;   // + staging of the epilogue warps
  auto kern = gemm_bf16_kernel<BN, STAGES, 2>;
  r = opt_in_smem(kern, smem); if (r) return r;
  const int tiles = (M / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, 192, smem, stream>>>(tmA, tmA, tmA, tmB, nullptr, M, N, K, N, 0, status, ca, GroupArgs{});
  return launch_result();
}

