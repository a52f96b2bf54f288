// Prefill attention on 5th-generation tensor cores: paged KV, 128-dim heads, GQA, causal / sliding-window /
// bidirectional masks, chunked prefill (query rows are the last q_len positions of a context of ctx_len).
//
// One CTA per (sequence, query head, tile of 128 query rows). Both contractions run as tcgen05.mma with
// FP32 accumulators in tensor memory:
//
//   S = Q Kᵀ      A = Q tile  [128 rows x 128 d]   (K-major, two 64-column blocks, 128-byte swizzle, TMA)
//                 B = K tile  [128 keys x 128 d]   (K-major, two pages of the cache, TMA)
//                 D = S       TMEM, 128 lanes x 128 columns, double-buffered so that Q K(j+1)ᵀ runs while the
//                             softmax warps work on tile j
//   O += P V      A = P tile  [128 rows x 128 keys] BF16, written by the softmax warps into 128-byte-swizzled
//                             shared memory (K-major over keys)
//                 B = V tile  [128 keys x 128 d]    exactly as the cache stores it: d contiguous = MN-major
//                 D = O       TMEM, 128 lanes x 128 columns, lives across all KV tiles
//
// Warp roles: warp 0 = TMA producer (Q once, then K tiles through a ring of two and V tiles through a ring of three
// stages -- a K tile is released right after its Q Kᵀ, so the loads run two tiles ahead; block ids read from the
// block table), warp 1 = MMA issuer, warps 2-9 = softmax: two threads share query row t (TMEM lane t) and split its
// key columns in halves (two warps per lane quadrant, so each scheduler has two warps to interleave); a thread reads its S
// row with tcgen05.ld, applies the mask where a tile needs one, keeps the running maximum and sum in the base-2 domain
// (scale folded into the exponent's FMA, ex2.approx straight on the MUFU), and
// rescales O in TMEM only when the maximum has moved by more than 2^8 (the stale maximum stays exact: P and
// the sum use the same reference, the final division cancels it).
//
// Every wait is bounded; a time-out records FF_ERR_TIMEOUT and the CTA leaves through the abort flag, frees
// its tensor memory and returns. Replaces the mma.sync prefill kernel of attention_paged.cu (kept for
// comparison) and the reference's FlashAttention-2 adapter / Rust-PTX prefill kernels
// (third_party/flash-attention/adapter.cu:147-162, device/src/lib.rs:422-940).
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr int TC_HD = 128, TC_PAGE = 64, TC_BM = 128, TC_BN = 128;
constexpr int TC_KSTAGES = 3, TC_VSTAGES = 3;             // K is done with after Q Kᵀ, V only after P V: separate rings
constexpr int TC_Q_BYTES = TC_BM * TC_HD * 2;             // 32 KiB
constexpr int TC_KV_BYTES = TC_BN * TC_HD * 2;            // 32 KiB per operand per stage
constexpr int TC_SMEM = TC_Q_BYTES + (TC_KSTAGES + TC_VSTAGES) * TC_KV_BYTES + 1024;   // 225 KiB
constexpr float TC_RESCALE_THRESHOLD = 8.0f;              // log2 units
constexpr int TC_TWO_CTAS_DEFAULT = 1;
constexpr int TC2_SPLIT_DEFAULT = 1;

struct alignas(8) TcBars {
  uint64_t q_full;
  uint64_t k_full[TC_KSTAGES];
  uint64_t k_empty[TC_KSTAGES];
  uint64_t v_full[TC_VSTAGES];
  uint64_t v_empty[TC_VSTAGES];
  uint64_t s_full[2];
  uint64_t s_empty[2];
  uint64_t p_full;
  uint64_t p_empty;
  uint64_t o_done;
  uint32_t tmem_base;
  int abort_flag;
  float xmax[2][TC_BM];      // row maxima (and, at the end, row sums) exchanged between the two warps of a quadrant
};

__global__ void __launch_bounds__(320, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const int* __restrict__ block_table,
                       const int* __restrict__ q_start, const int* __restrict__ q_lens,
                       const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, int hq, int hkv, int ldo,
                       int max_blocks, int num_blocks, float scale_log2, int window, int causal, int* status,
                       const float* __restrict__ sinks) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int qlen = q_lens[b];
  // later query tiles of a causal prefill see more keys: they are scheduled first so that the long CTAs do not form the tail
  const int r0 = (gridDim.x - 1 - blockIdx.x) * TC_BM;
  if (r0 >= qlen) return;
  extern __shared__ uint8_t smem_raw[];
  __shared__ TcBars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKr = smem + TC_Q_BYTES;                       // K ring, then V ring: 32 KiB tiles
  uint8_t* sVr = sKr + TC_KSTAGES * TC_KV_BYTES;
  const int ctx = ctx_lens[b], qs = q_start[b];
  const int kvh = h / (hq / hkv);
  const int past = ctx - qlen;
  const int real = min(TC_BM, qlen - r0);
  // key range of this tile
  const int last_key = causal ? past + r0 + real - 1 : ctx - 1;
  const int first_key = window > 0 ? max(0, past + r0 - window + 1) : 0;
  const int t0 = first_key / TC_BN, t1 = last_key / TC_BN + 1;
  const int ntiles = t1 - t0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(&bars.q_full, 1);
    for (int i = 0; i < TC_KSTAGES; ++i) { mbar_init(&bars.k_full[i], 1); mbar_init(&bars.k_empty[i], 1); }
    for (int i = 0; i < TC_VSTAGES; ++i) { mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars.s_full[i], 1); mbar_init(&bars.s_empty[i], 8); }
    mbar_init(&bars.p_full, 1); mbar_init(&bars.p_empty, 1); mbar_init(&bars.o_done, 1);
    bars.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  const uint32_t tmem_o = tmem_base + 256;
  const uint32_t tmem_p = tmem_base + 384;       // P: 128 keys as 64 columns of packed BF16 pairs
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      mbar_expect_tx(&bars.q_full, TC_Q_BYTES);
      // rows past the sequence's own belong to the next sequence of the packed batch (or are out of range and read
      // as zero): their lanes are computed and never stored
      tma_load_2d(sQ, &tmQ, &bars.q_full, h * TC_HD, qs + r0);
      tma_load_2d(sQ + TC_BM * 128, &tmQ, &bars.q_full, h * TC_HD + 64, qs + r0);
      bool ok = true, bad = false;
      const int nblk = (ctx + TC_PAGE - 1) / TC_PAGE;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int ks = j % TC_KSTAGES, vs = j % TC_VSTAGES;
        int rows[2];
        for (int pg = 0; pg < 2; ++pg) {
          int page = (t0 + j) * 2 + pg;
          if (page >= nblk) page = nblk - 1;                 // past the context: any valid page, its keys are masked
          int blk = block_table[(size_t)b * max_blocks + page];
          if (blk < 0 || blk >= num_blocks) { bad = true; blk = 0; }
          rows[pg] = (blk * hkv + kvh) * TC_PAGE;
        }
        // layout of a tile: block d0 = [128 keys x 64 d] (16 KiB), then block d1; a page is 64 keys of each
        if (!mbar_wait(&bars.k_empty[ks], ((j / TC_KSTAGES) & 1) ^ 1, abort_flag, status, KID_ATTN_PREFILL, 1)) { ok = false; break; }
        mbar_expect_tx(&bars.k_full[ks], TC_KV_BYTES);
        uint8_t* sK = sKr + ks * TC_KV_BYTES;
        for (int pg = 0; pg < 2; ++pg) {
          tma_load_2d(sK + pg * 8192, &tmK, &bars.k_full[ks], 0, rows[pg]);
          tma_load_2d(sK + 16384 + pg * 8192, &tmK, &bars.k_full[ks], 64, rows[pg]);
        }
        if (!mbar_wait(&bars.v_empty[vs], ((j / TC_VSTAGES) & 1) ^ 1, abort_flag, status, KID_ATTN_PREFILL, 10)) { ok = false; break; }
        mbar_expect_tx(&bars.v_full[vs], TC_KV_BYTES);
        uint8_t* sV = sVr + vs * TC_KV_BYTES;
        for (int pg = 0; pg < 2; ++pg) {
          tma_load_2d(sV + pg * 8192, &tmV, &bars.v_full[vs], 0, rows[pg]);
          tma_load_2d(sV + 16384 + pg * 8192, &tmV, &bars.v_full[vs], 64, rows[pg]);
        }
      }
      if (bad) set_status(status, KID_ATTN_PREFILL, FF_ERR_BOUNDS, b, r0 / TC_BM);
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, 0, 0, TC_BM, TC_BN);      // Q (K-major) x K (K-major)
      const uint32_t idesc_o = umma_idesc(1, 1, 0, 1, TC_BM, TC_HD);      // P (K-major) x V (MN-major)
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(&bars.q_full, 0, abort_flag, status, KID_ATTN_PREFILL, 2);
      auto issue_s = [&](int j) -> bool {
        const int ks = j % TC_KSTAGES; const uint32_t ph = (j / TC_KSTAGES) & 1;
        const int sb = j & 1; const uint32_t sph = (j >> 1) & 1;
        if (!mbar_wait(&bars.k_full[ks], ph, abort_flag, status, KID_ATTN_PREFILL, 3)) return false;
        if (!mbar_wait(&bars.s_empty[sb], sph ^ 1, abort_flag, status, KID_ATTN_PREFILL, 4)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKr + ks * TC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(tmem_base + sb * TC_BN, umma_desc_sw128(q_addr + off, 16, 1024), umma_desc_sw128(k_addr + off, 16, 1024),
                   idesc_s, k != 0);
        }
        umma_commit(&bars.s_full[sb]);
        umma_commit(&bars.k_empty[ks]);            // the K tile is free as soon as this product has read it
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) { ok = issue_s(j + 1); if (!ok) break; }
        if (!mbar_wait(&bars.p_full, j & 1, abort_flag, status, KID_ATTN_PREFILL, 5)) { ok = false; break; }
        const int vs = j % TC_VSTAGES;
        if (!mbar_wait(&bars.v_full[vs], (j / TC_VSTAGES) & 1, abort_flag, status, KID_ATTN_PREFILL, 11)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sVr + vs * TC_KV_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // P: the 16 keys of k-step k are 8 columns of the P region of tensor memory; V: 16 key rows = 2 KiB
          const uint64_t db = umma_desc_sw128(v_addr + (k >> 2) * 8192 + (k & 3) * 2048, 16384, 1024);
          umma_f16_ts(tmem_o, tmem_p + k * 8, db, idesc_o, (j > 0) || (k != 0));
        }
        umma_commit(&bars.p_empty);
        umma_commit(&bars.v_empty[vs]);
      }
      if (ok) umma_commit(&bars.o_done);
    }
  } else {
    // ================================ softmax warps 2..9 ================================
    // Two warps per 32-lane quadrant of tensor memory (a warp may only touch the lanes of quadrant warp % 4): the pair
    // shares the rows of its quadrant and splits a tile's 128 key columns (and O's 128 columns, when it is rescaled)
    // in halves, so every scheduler has two warps to interleave. Row maxima cross the pair through shared memory.
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;               // which 64-column half this warp owns
    const int row = q * 32 + lane;                // query row of the tile = TMEM lane
    const int e = (warp - 2) * 32 + lane;
    const bool live = row < real;
    const int pos = past + r0 + row;              // absolute position of the row
    const int hi = live ? (causal ? pos : ctx - 1) : -1;
    const int lo = (live && window > 0) ? max(0, pos - window + 1) : 0;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    const uint32_t lane_base = (uint32_t(q * 32) << 16);
    // key range common to all live rows of the tile: [largest lower bound, smallest upper bound]
    const int tile_hi_min = causal ? past + r0 : ctx - 1;
    const int tile_lo_max = window > 0 ? max(0, past + r0 + real - window) : 0;
    constexpr int HB = TC_BN / 2;                 // columns per warp
    // A wait that gives up clears `ok` for the whole warp; the warp then skips the work of the remaining tiles but still
    // takes part in every barrier, so that no other warp is left waiting for it.
    for (int j = 0; j < ntiles; ++j) {
      const int sb = j & 1; const uint32_t sph = (j >> 1) & 1;
      if (ok && !mbar_wait(&bars.s_full[sb], sph, abort_flag, status, KID_ATTN_PREFILL, 6)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      float sv[HB];
      float mx = -INFINITY;
      if (ok) {
      tc_fence_after();
      {
        uint32_t r[HB];
#pragma unroll
        for (int c = 0; c < HB; c += 32) tmem_ld_x32(tmem_base + lane_base + sb * TC_BN + hf * HB + c, r + c);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < HB; ++i) sv[i] = __uint_as_float(r[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.s_empty[sb]);
      const int k0 = (t0 + j) * TC_BN + hf * HB;
      // sv stays in raw score units: the scale is folded into the exponent's FMA below. A tile that lies inside the key
      // range of every live row of this query tile (most tiles of a long context) skips the mask altogether.
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if ((t0 + j) * TC_BN >= tile_lo_max && (t0 + j) * TC_BN + TC_BN - 1 <= tile_hi_min) {
#pragma unroll
        for (int i = 0; i < HB; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
      } else {
#pragma unroll
        for (int i = 0; i < HB; ++i) {
          const int key = k0 + i;
          const float t = (key >= lo && key <= hi) ? sv[i] : -INFINITY;
          sv[i] = t;
          mx4[i & 3] = fmaxf(mx4[i & 3], t);
        }
      }
      mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale > 0 commutes with the maximum
      }
      // the row's maximum over both halves: through shared memory, one 64-thread barrier per quadrant pair
      bars.xmax[hf][row] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
      mx = fmaxf(mx, bars.xmax[hf ^ 1][row]);
      // the previous P V must be done before P is overwritten or O is rescaled
      if (ok && !mbar_wait(&bars.p_empty, (j & 1) ^ 1, abort_flag, status, KID_ATTN_PREFILL, 7)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
      tc_fence_after();
      float alpha = 1.f;
      bool need = false;
      if (mx > m_ref + TC_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY)) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
        need = j > 0;                              // O holds nothing before the first P V
      }
      if (__any_sync(0xffffffffu, need)) {
        // rescale this warp's half of the 32 lanes of O (lanes that did not move keep alpha = 1)
#pragma unroll
        for (int c = 0; c < TC_HD / 2; c += 16) {
          uint32_t r[16];
          tmem_ld_x16(tmem_o + lane_base + hf * (TC_HD / 2) + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_x16(tmem_o + lane_base + hf * (TC_HD / 2) + c, r);
        }
        tmem_st_wait();
      }
      l_sum *= alpha;
      // P = 2^(s * scale - m_ref), BF16, into 128-byte-swizzled K-major shared memory: row `row`, 16-byte chunk c of 64-key
      // block kb (= this warp's half) at (row / 8) * 1024 + (row % 8) * 128 + ((c ^ (row % 8)) * 16)
      const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[HB / 2];
#pragma unroll
      for (int i = 0; i < HB / 2; ++i) {
        // one FMA and one MUFU per value; a masked score is -inf and gives exactly 0
        const float p0 = ex2_approx(fmaf(sv[2 * i], scale_log2, -mr));
        const float p1 = ex2_approx(fmaf(sv[2 * i + 1], scale_log2, -mr));
        pk[i] = pack_bf16x2(p0, p1);
        ls4[i & 3] += p0 + p1;
      }
      // P stays in tensor memory: row = lane, two BF16 keys per 32-bit column, this warp's 64 keys = 32 columns; the second
      // product reads it from there as its A operand (no trip through shared memory, whose bandwidth the two products'
      // operand reads already use up)
      tmem_st_x16(tmem_p + lane_base + hf * (HB / 2), pk);
      tmem_st_x16(tmem_p + lane_base + hf * (HB / 2) + 16, pk + 16);
      tmem_st_wait();
      l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      tc_fence_before();
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (e == 0 && ok) mbar_arrive(&bars.p_full);
    }
    if (ok) ok = mbar_wait(&bars.o_done, 0, abort_flag, status, KID_ATTN_PREFILL, 8);
    ok = __all_sync(0xffffffffu, ok);
    // the row's sum over both halves
    bars.xmax[hf][row] = l_sum;
    asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
    if (ok) {
      tc_fence_after();
      l_sum += bars.xmax[hf ^ 1][row];
      // learnable soft-max: one extra logit per head that enters the denominator only
      if (sinks != nullptr) l_sum += (m_ref == -INFINITY) ? 1.f : exp2f(sinks[h] * 1.4426950408889634f - m_ref);
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = out + (size_t)(qs + r0 + row) * ldo + (size_t)h * TC_HD + hf * (TC_HD / 2);
#pragma unroll
      for (int c = 0; c < TC_HD / 2; c += 16) {
        uint32_t r[16];
        tmem_ld_x16(tmem_o + lane_base + hf * (TC_HD / 2) + c, r);
        tmem_ld_wait();
        if (live) {
          uint4 o0, o1;
          o0.x = pack_bf16x2(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          o0.y = pack_bf16x2(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          o0.z = pack_bf16x2(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          o0.w = pack_bf16x2(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          o1.x = pack_bf16x2(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
          o1.y = pack_bf16x2(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
          o1.z = pack_bf16x2(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
          o1.w = pack_bf16x2(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
          *reinterpret_cast<uint4*>(orow + c) = o0;
          *reinterpret_cast<uint4*>(orow + c + 8) = o1;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0w = globaltimer_ns();
    while (globaltimer_ns() - t0w < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}


// ------------------------------------------------------------------------------------------------
// Two CTAs per SM, 64-key tiles. The same products and masks, arranged so that two CTAs fit one SM and every role runs
// ahead of the next: per CTA 97 KB of shared memory (Q, two K tiles and two V tiles of one 64-key page each), 256 columns
// of tensor memory (two S buffers of 64 columns and O; P is written over the first 32 columns of the S buffer it came
// from, by the thread that owns the row, after it has taken its S values into registers), 6 warps (TMA, MMA, one softmax
// warp per lane quadrant, a thread owning a row). Q K(j+1)ᵀ is issued as soon as its K page is there, i.e. while the
// softmax warps are still on tile j; P V(j) runs while they are on tile j + 1; only the rare rescale of O waits for the
// previous P V. FF_ATTN_PREFILL_SPLIT=2 puts two softmax warps on every lane quadrant (32 columns each).
// ------------------------------------------------------------------------------------------------
constexpr int T2_BN = 64;                                          // keys per tile = one cache page
constexpr int T2_KV_BYTES = T2_BN * TC_HD * 2;                     // 16 KiB
constexpr int TC2_SMEM = TC_Q_BYTES + 4 * T2_KV_BYTES + 1024;      // 97 KiB

struct alignas(8) Tc2Bars {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pv_done[2];
  uint32_t tmem_base;
  int abort_flag;
  float xmax[2][TC_BM];
};

template <int SPLIT>
__global__ void __launch_bounds__(64 + 128 * SPLIT, 2)
attn_prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const int* __restrict__ block_table,
                        const int* __restrict__ q_start, const int* __restrict__ q_lens,
                        const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, int hq, int hkv, int ldo,
                        int max_blocks, int num_blocks, float scale_log2, int window, int causal, int* status,
                        const float* __restrict__ sinks) {
  const int b = blockIdx.z, h = blockIdx.y;
  const int qlen = q_lens[b];
  const int r0 = (gridDim.x - 1 - blockIdx.x) * TC_BM;            // long (late) query tiles first
  if (r0 >= qlen) return;
  extern __shared__ uint8_t smem_raw[];
  __shared__ Tc2Bars bars;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + TC_Q_BYTES;                                 // two K tiles, then two V tiles
  uint8_t* sV = sK + 2 * T2_KV_BYTES;
  const int ctx = ctx_lens[b], qs = q_start[b];
  const int kvh = h / (hq / hkv);
  const int past = ctx - qlen;
  const int real = min(TC_BM, qlen - r0);
  const int last_key = causal ? past + r0 + real - 1 : ctx - 1;
  const int first_key = window > 0 ? max(0, past + r0 - window + 1) : 0;
  const int t0 = first_key / T2_BN, t1 = last_key / T2_BN + 1;
  const int ntiles = t1 - t0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_init(&bars.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars.k_full[i], 1); mbar_init(&bars.k_empty[i], 1); mbar_init(&bars.v_full[i], 1); mbar_init(&bars.v_empty[i], 1);
      mbar_init(&bars.s_full[i], 1); mbar_init(&bars.p_full[i], 1); mbar_init(&bars.pv_done[i], 1);
    }
    bars.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = bars.tmem_base;          // S buffer i: columns 64 i .. 64 i + 63; its P over the first 32 of them
  const uint32_t tmem_o = bars.tmem_base + 128;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(&bars.q_full, TC_Q_BYTES);
      tma_load_2d(sQ, &tmQ, &bars.q_full, h * TC_HD, qs + r0);
      tma_load_2d(sQ + TC_BM * 128, &tmQ, &bars.q_full, h * TC_HD + 64, qs + r0);
      bool ok = true, bad = false;
      const int nblk = (ctx + TC_PAGE - 1) / TC_PAGE;
      auto tile_row = [&](int j) -> int {
        int page = t0 + j;
        if (page >= nblk) page = nblk - 1;                   // past the context: any valid page, its keys are masked
        int blk = block_table[(size_t)b * max_blocks + page];
        if (blk < 0 || blk >= num_blocks) { bad = true; blk = 0; }
        return (blk * hkv + kvh) * TC_PAGE;
      };
      // a tile: block d0 = [64 keys x 64 d] (8 KiB), then block d1. K runs one tile ahead of V: K(j + 1) is free once
      // Q K(j - 1) has run, V(j) only once P V(j - 2) has.
      auto load_k = [&](int j) -> bool {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        const int row = tile_row(j);
        if (!mbar_wait(&bars.k_empty[st], ph ^ 1, abort_flag, status, KID_ATTN_PREFILL, 21)) return false;
        mbar_expect_tx(&bars.k_full[st], T2_KV_BYTES);
        tma_load_2d(sK + st * T2_KV_BYTES, &tmK, &bars.k_full[st], 0, row);
        tma_load_2d(sK + st * T2_KV_BYTES + 8192, &tmK, &bars.k_full[st], 64, row);
        return true;
      };
      ok = load_k(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles && !load_k(j + 1)) { ok = false; break; }
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        const int row = tile_row(j);
        if (!mbar_wait(&bars.v_empty[st], ph ^ 1, abort_flag, status, KID_ATTN_PREFILL, 22)) { ok = false; break; }
        mbar_expect_tx(&bars.v_full[st], T2_KV_BYTES);
        tma_load_2d(sV + st * T2_KV_BYTES, &tmV, &bars.v_full[st], 0, row);
        tma_load_2d(sV + st * T2_KV_BYTES + 8192, &tmV, &bars.v_full[st], 64, row);
      }
      if (bad) set_status(status, KID_ATTN_PREFILL, FF_ERR_BOUNDS, b, r0 / TC_BM);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(1, 1, 0, 0, TC_BM, T2_BN);
      const uint32_t idesc_o = umma_idesc(1, 1, 0, 1, TC_BM, TC_HD);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(&bars.q_full, 0, abort_flag, status, KID_ATTN_PREFILL, 23);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars.k_full[st], ph, abort_flag, status, KID_ATTN_PREFILL, 24)) return false;
        // this S buffer still holds the P of tile j - 2: that tile's P V has to be complete
        if (j >= 2 && !mbar_wait(&bars.pv_done[st], ph ^ 1, abort_flag, status, KID_ATTN_PREFILL, 25)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sK + st * T2_KV_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // Q: 64-column block k / 4 of a 128-row tile (16 KiB), 32 bytes per k-step; K: the same with 64 rows (8 KiB)
          umma_f16(tmem_s + st * T2_BN, umma_desc_sw128(q_addr + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                   umma_desc_sw128(k_addr + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), idesc_s, k != 0);
        }
        umma_commit(&bars.s_full[st]);
        umma_commit(&bars.k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < ntiles && ok; ++j) {
        if (j + 1 < ntiles) { ok = issue_s(j + 1); if (!ok) break; }
        const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&bars.p_full[st], ph, abort_flag, status, KID_ATTN_PREFILL, 26)) { ok = false; break; }
        if (!mbar_wait(&bars.v_full[st], ph, abort_flag, status, KID_ATTN_PREFILL, 27)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * T2_KV_BYTES);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // P: 16 keys = 8 columns of packed pairs; V: 16 key rows = 2 KiB inside each 64-dim block, blocks 8 KiB apart
          umma_f16_ts(tmem_o, tmem_s + st * T2_BN + k * 8, umma_desc_sw128(v_addr + k * 2048, 8192, 1024), idesc_o,
                      (j > 0) || (k != 0));
        }
        umma_commit(&bars.pv_done[st]);
        umma_commit(&bars.v_empty[st]);
      }
    }
  } else {
    constexpr int HB = T2_BN / SPLIT;             // columns of a tile per thread
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;
    const int row = q * 32 + lane;
    const int e = (warp - 2) * 32 + lane;
    const bool live = row < real;
    const int pos = past + r0 + row;
    const int hi = live ? (causal ? pos : ctx - 1) : -1;
    const int lo = (live && window > 0) ? max(0, pos - window + 1) : 0;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    const uint32_t lane_base = (uint32_t(q * 32) << 16);
    const int tile_hi_min = causal ? past + r0 : ctx - 1;
    const int tile_lo_max = window > 0 ? max(0, past + r0 + real - window) : 0;
    for (int j = 0; j < ntiles; ++j) {
      const int st = j & 1; const uint32_t ph = (j >> 1) & 1;
      if (ok && !mbar_wait(&bars.s_full[st], ph, abort_flag, status, KID_ATTN_PREFILL, 28)) ok = false;
      ok = __all_sync(0xffffffffu, ok);
      float sv[HB];
      float mx = -INFINITY;
      const uint32_t s_addr = tmem_s + lane_base + st * T2_BN;
      if (ok) {
        tc_fence_after();
        {
          uint32_t r[HB];
          if (HB == 64) { tmem_ld_x32(s_addr, r); tmem_ld_x32(s_addr + 32, r + 32); }
          else tmem_ld_x32(s_addr + hf * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < HB; ++i) sv[i] = __uint_as_float(r[i]);
        }
        const int k0 = (t0 + j) * T2_BN + hf * HB;
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if ((t0 + j) * T2_BN >= tile_lo_max && (t0 + j) * T2_BN + T2_BN - 1 <= tile_hi_min) {
#pragma unroll
          for (int i = 0; i < HB; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], sv[i]);
        } else {
#pragma unroll
          for (int i = 0; i < HB; ++i) {
            const int key = k0 + i;
            const float t = (key >= lo && key <= hi) ? sv[i] : -INFINITY;
            sv[i] = t;
            mx4[i & 3] = fmaxf(mx4[i & 3], t);
          }
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      }
      if (SPLIT == 2) {
        // after this barrier both warps of the pair hold their S columns in registers: P may overwrite S
        bars.xmax[hf][row] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
        mx = fmaxf(mx, bars.xmax[hf ^ 1][row]);
      }
      float alpha = 1.f;
      bool need = false;
      if (ok && (mx > m_ref + TC_RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY))) {
        alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - mx);
        m_ref = mx;
        need = j > 0;
      }
      if (__any_sync(0xffffffffu, need)) {
        // O is rescaled in place: the P V of the previous tile has to be complete (the rare path)
        if (ok && !mbar_wait(&bars.pv_done[st ^ 1], ((j - 1) >> 1) & 1, abort_flag, status, KID_ATTN_PREFILL, 30)) ok = false;
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < TC_HD / SPLIT; c += 16) {
            uint32_t r[16];
            tmem_ld_x16(tmem_o + lane_base + hf * (TC_HD / SPLIT) + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_x16(tmem_o + lane_base + hf * (TC_HD / SPLIT) + c, r);
          }
          tmem_st_wait();
        }
      }
      if (ok) {
        l_sum *= alpha;
        const float mr = (m_ref == -INFINITY) ? 0.f : m_ref;
        float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < HB / 2; c += 16) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float p0 = ex2_approx(fmaf(sv[2 * (c + i)], scale_log2, -mr));
            const float p1 = ex2_approx(fmaf(sv[2 * (c + i) + 1], scale_log2, -mr));
            pk[i] = pack_bf16x2(p0, p1);
            ls4[i & 3] += p0 + p1;
          }
          // P over the first 32 columns of this S buffer: the thread's own lane, whose S values are in registers by now
          tmem_st_x16(s_addr + hf * (HB / 2) + c, pk);
        }
        tmem_st_wait();
        l_sum += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
        tc_fence_before();
      }
      // one arrival for the whole tile; an arrival per warp (no common barrier) measured 1.5 % slower
      if (SPLIT == 2) asm volatile("bar.sync 1, 256;" ::: "memory");
      else asm volatile("bar.sync 1, 128;" ::: "memory");
      if (e == 0 && ok) mbar_arrive(&bars.p_full[st]);
    }
    // the last P V
    if (ok && !mbar_wait(&bars.pv_done[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1, abort_flag, status, KID_ATTN_PREFILL, 29)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    if (SPLIT == 2) {
      bars.xmax[hf][row] = l_sum;
      asm volatile("bar.sync %0, 64;" ::"r"(2 + q) : "memory");
      l_sum += bars.xmax[hf ^ 1][row];
    }
    if (ok) {
      tc_fence_after();
      if (sinks != nullptr) l_sum += (m_ref == -INFINITY) ? 1.f : exp2f(sinks[h] * 1.4426950408889634f - m_ref);
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* orow = out + (size_t)(qs + r0 + row) * ldo + (size_t)h * TC_HD + hf * (TC_HD / SPLIT);
#pragma unroll
      for (int c = 0; c < TC_HD / SPLIT; c += 16) {
        uint32_t r[16];
        tmem_ld_x16(tmem_o + lane_base + hf * (TC_HD / SPLIT) + c, r);
        tmem_ld_wait();
        if (live) {
          uint4 o0, o1;
          o0.x = pack_bf16x2(__uint_as_float(r[0]) * inv, __uint_as_float(r[1]) * inv);
          o0.y = pack_bf16x2(__uint_as_float(r[2]) * inv, __uint_as_float(r[3]) * inv);
          o0.z = pack_bf16x2(__uint_as_float(r[4]) * inv, __uint_as_float(r[5]) * inv);
          o0.w = pack_bf16x2(__uint_as_float(r[6]) * inv, __uint_as_float(r[7]) * inv);
          o1.x = pack_bf16x2(__uint_as_float(r[8]) * inv, __uint_as_float(r[9]) * inv);
          o1.y = pack_bf16x2(__uint_as_float(r[10]) * inv, __uint_as_float(r[11]) * inv);
          o1.z = pack_bf16x2(__uint_as_float(r[12]) * inv, __uint_as_float(r[13]) * inv);
          o1.w = pack_bf16x2(__uint_as_float(r[14]) * inv, __uint_as_float(r[15]) * inv);
          *reinterpret_cast<uint4*>(orow + c) = o0;
          *reinterpret_cast<uint4*>(orow + c + 8) = o1;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0w = globaltimer_ns();
    while (globaltimer_ns() - t0w < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(bars.tmem_base, 256); }
}

}  // namespace ff
using namespace ff;

// Same contract as ff_attn_prefill (attention_paged.cu). q: packed rows [rows, ldq] with head h at columns h*128;
// out rows 16-byte aligned (ldo % 8 == 0). window > 0 sliding, 0 causal, < 0 bidirectional.
FF_EXPORT int ff_attn_prefill_tc(const void* q, const void* kcache, const void* vcache, const int* block_table,
                                 const int* q_start, const int* q_lens, const int* ctx_lens, void* out, int batch,
                                 int total_rows, int max_q_len, int hq, int hkv, int head_dim, int ldq, int ldo,
                                 int max_blocks, int num_blocks, float scale, int window, const float* sinks, int* status,
                                 cudaStream_t s) {
  if (head_dim != TC_HD || batch <= 0 || max_q_len <= 0 || hq <= 0 || hkv <= 0 || hq % hkv || total_rows <= 0) return FF_HOST_BAD_SHAPE;
  if (ldq % 8 || ldo % 8 || (reinterpret_cast<uintptr_t>(out) & 15)) return FF_HOST_BAD_ALIGN;
  CUtensorMap tmQ, tmK, tmV;
  if (int r = make_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)ldq, (uint64_t)total_rows,
                           (uint64_t)ldq * 2, 64, TC_BM)) return r;
  const uint64_t cache_rows = (uint64_t)num_blocks * hkv * TC_PAGE;
  if (int r = make_tmap_2d(&tmK, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, TC_HD, cache_rows, TC_HD * 2, 64, TC_PAGE)) return r;
  if (int r = make_tmap_2d(&tmV, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, TC_HD, cache_rows, TC_HD * 2, 64, TC_PAGE)) return r;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((max_q_len + TC_BM - 1) / TC_BM, hq, batch);
  // FF_ATTN_PREFILL_CTAS = 1 selects the one-CTA-per-SM kernel (deep K / V rings, eight softmax warps); the default is the
  // two-CTAs-per-SM kernel
  static int two = -1;
  if (two < 0) { const char* e = getenv("FF_ATTN_PREFILL_CTAS"); two = (e != nullptr && e[0] == '1') ? 0 : TC_TWO_CTAS_DEFAULT; }
  if (two) {
    // FF_ATTN_PREFILL_SPLIT = 2: two softmax warps per lane quadrant (64 columns each) instead of one
    static int split = -1;
    if (split < 0) { const char* e = getenv("FF_ATTN_PREFILL_SPLIT"); split = (e != nullptr && (e[0] == '1' || e[0] == '2')) ? e[0] - '0' : TC2_SPLIT_DEFAULT; }
    if (split == 2) {
      if (int r = opt_in_smem(attn_prefill_tc2_kernel<2>, TC2_SMEM)) return r;
      attn_prefill_tc2_kernel<2><<<grid, 320, TC2_SMEM, s>>>(tmQ, tmK, tmV, block_table, q_start, q_lens, ctx_lens,
                                                             (__nv_bfloat16*)out, hq, hkv, ldo, max_blocks, num_blocks, scale_log2,
                                                             window < 0 ? 0 : window, window < 0 ? 0 : 1, status, sinks);
      return launch_result();
    }
    if (int r = opt_in_smem(attn_prefill_tc2_kernel<1>, TC2_SMEM)) return r;
    attn_prefill_tc2_kernel<1><<<grid, 192, TC2_SMEM, s>>>(tmQ, tmK, tmV, block_table, q_start, q_lens, ctx_lens,
                                                           (__nv_bfloat16*)out, hq, hkv, ldo, max_blocks, num_blocks, scale_log2,
                                                           window < 0 ? 0 : window, window < 0 ? 0 : 1, status, sinks);
    return launch_result();
  }
  if (int r = opt_in_smem(attn_prefill_tc_kernel, TC_SMEM)) return r;
  attn_prefill_tc_kernel<<<grid, 320, TC_SMEM, s>>>(tmQ, tmK, tmV, block_table, q_start, q_lens, ctx_lens,
                                                    (__nv_bfloat16*)out, hq, hkv, ldo, max_blocks, num_blocks, scale_log2,
                                                    window < 0 ? 0 : window, window < 0 ? 0 : 1, status, sinks);
  return launch_result();
}
