// Paged GQA attention (head_dim 128) over the block cache written by rope_kv_paged:
//   attn_decode : split-KV flash-decode. One CTA = (split, kv head, sequence); the G query heads of
//                 the group (times up to 16/G query rows for multi-row verification) are packed
//                 into one 16-row MMA tile so each K/V byte is read once per group. Partials
//                 (m, l, acc) go to scratch and a merge kernel combines the splits; with one
//                 split the CTA writes the output directly.
//   attn_prefill: causal chunked prefill. One CTA = (64-row query tile, q head, sequence); K/V
//                 pages stream through a cp.async double buffer shared by the four warps.
// Both are bandwidth / latency bound at the shapes served here (decode) or a few percent of
// the layer's FLOPs (prefill at 1k-8k tokens), so they use register-level mma.sync tiles whose
// operands come straight from the 64-token pages; softmax is FP32 online with a finite
// running-max sentinel, like the reference's flash-decode (kernels/attention.cu:138-397) and
// its multi-query verify variant (kernels/attention.cu:598-616).
// Optional per-row visibility: `tree_mask` gives each query row a 64-bit ancestor set over
// the last `nq` positions (tree speculation, kernels/tcmqa.cu:1-75); without it rows are
// causal.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int HD = 128;             // head dim
constexpr int PAGE = 64;            // tokens per cache block
#ifndef DEC_WARPS
#define DEC_WARPS 4                 // decode attention: warps per CTA (keys per warp = 64 / DEC_WARPS)
#endif
#ifndef DEC_STAGES
#define DEC_STAGES 2                // decode attention: pages in flight per CTA + 1
#endif
constexpr float NEG_BIG = -3.0e38f;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A 64-row page tile [64][128] bf16 sits in shared memory as two halves of 64 dims, each [64 rows][128 bytes]
// with the 16-byte chunk index XORed by row % 8: exactly what a TMA load of a {64 dims, 64 rows} box
// with 128-byte swizzle writes, so the same tile can come from cp.async or from TMA.
// Byte offset of 16-byte chunk `c` (0..15) of row `r`:
__device__ __forceinline__ uint32_t tile_off(int r, int c) {
  return (uint32_t)((c >> 3) * (PAGE * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// copy one page slice [nrows][128] bf16 from global to a swizzled smem tile, all `nthreads` threads
__device__ __forceinline__ void load_tile_async(uint8_t* stile, const __nv_bfloat16* gsrc, int nrows, int tid,
                                                int nthreads) {
  for (int i = tid; i < nrows * 16; i += nthreads) {
    const int r = i >> 4, c = i & 15;
    cp_async16(stile + tile_off(r, c), gsrc + (size_t)r * HD + c * 8);
  }
}

// State of one warp's 16 query rows.
struct RowState {
  float m[2], l[2];
  float o[16][4];
};

// One warp consumes NT8 n-tiles (8 keys each) starting at smem row key_off.
//   qf        : Q fragments for the 8 k-steps
//   key0      : global key index of smem row key_off
//   lim0/lim1 : last visible key index for rows g and g+8 (inclusive); mask0/mask1: optional
//               64-bit ancestor sets over keys >= tail_start (bit i = key tail_start+i visible)
template <int NT8>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[8][4], RowState& st, uint32_t sK, uint32_t sV,
                                          int key_off, int key0, int lim0, int lim1, bool use_mask, int tail_start,
                                          unsigned long long mask0, unsigned long long mask1, float scale_log2) {
  const int lane = threadIdx.x & 31, t = lane & 3;
  float s[NT8][4];
#pragma unroll
  for (int i = 0; i < NT8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
  // S = Q K^T
  // chunk = 2*kk + h with h = (lane >> 3) & 1: (chunk & 7) ^ (key & 7) = (2*(kk & 3)) ^ (h ^ (lane & 7))
  const uint32_t kbase = sK + (uint32_t)(key_off + ((lane >> 4) << 3) + (lane & 7)) * 128u;
  const uint32_t khx = ((lane >> 3) & 1) ^ (lane & 7);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
    for (int np = 0; np < NT8 / 2; ++np) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(kbase + (uint32_t)(np * 16 * 128 + (kk >> 2) * (PAGE * 128)) + (((uint32_t)(2 * (kk & 3)) ^ khx) << 4), b0, b1, b2, b3);
      mma_bf16(s[2 * np], qf[kk], b0, b1);
      mma_bf16(s[2 * np + 1], qf[kk], b2, b3);
    }
  }
  // mask + online softmax
  float mx0 = NEG_BIG, mx1 = NEG_BIG;
#pragma unroll
  for (int i = 0; i < NT8; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int key = key0 + i * 8 + 2 * t + (j & 1);
      const int lim = (j < 2) ? lim0 : lim1;
      bool vis = key <= lim;
      if (use_mask && key >= tail_start) {
        const unsigned long long mk = (j < 2) ? mask0 : mask1;
        vis = vis && ((mk >> (key - tail_start)) & 1ull);
      }
      const float v = vis ? s[i][j] * scale_log2 : NEG_BIG;
      s[i][j] = v;
      if (j < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
    }
  }
  mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
  mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
  const float mn0 = fmaxf(st.m[0], mx0), mn1 = fmaxf(st.m[1], mx1);
  const float a0 = exp2f(st.m[0] - mn0), a1 = exp2f(st.m[1] - mn1);
  st.m[0] = mn0; st.m[1] = mn1;
  float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
  for (int i = 0; i < NT8; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float mref = (j < 2) ? mn0 : mn1;
      const float p = (s[i][j] <= NEG_BIG) ? 0.f : exp2f(s[i][j] - mref);
      s[i][j] = p;
      if (j < 2) rs0 += p; else rs1 += p;
    }
  }
  st.l[0] = st.l[0] * a0 + rs0;   // per-thread partial row sums; quad-reduced at the end
  st.l[1] = st.l[1] * a1 + rs1;
  // the running maxima settle after the first tiles: skip the 64 multiplications by exactly 1
  if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) { st.o[i][0] *= a0; st.o[i][1] *= a0; st.o[i][2] *= a1; st.o[i][3] *= a1; }
  }
  // O += P V
#pragma unroll
  for (int ks = 0; ks < NT8 / 2; ++ks) {
    uint32_t pa[4];
    pa[0] = pack_bf16x2(s[2 * ks][0], s[2 * ks][1]);
    pa[1] = pack_bf16x2(s[2 * ks][2], s[2 * ks][3]);
    pa[2] = pack_bf16x2(s[2 * ks + 1][0], s[2 * ks + 1][1]);
    pa[3] = pack_bf16x2(s[2 * ks + 1][2], s[2 * ks + 1][3]);
    const uint32_t vbase = sV + (uint32_t)(key_off + ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * 128u;
    const uint32_t vhx = (lane >> 4) ^ (lane & 7);
#pragma unroll
    for (int dp = 0; dp < 8; ++dp) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vbase + (uint32_t)((dp >> 2) * (PAGE * 128)) + (((uint32_t)(2 * (dp & 3)) ^ vhx) << 4), b0, b1, b2, b3);
      mma_bf16(st.o[2 * dp], pa, b0, b1);
      mma_bf16(st.o[2 * dp + 1], pa, b2, b3);
    }
  }
}

__device__ __forceinline__ void init_state(RowState& st) {
  st.m[0] = st.m[1] = NEG_BIG; st.l[0] = st.l[1] = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) st.o[i][0] = st.o[i][1] = st.o[i][2] = st.o[i][3] = 0.f;
}

// Q fragments for rows (r0, r0+8) given per-row pointers (null -> zero row)
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[8][4], const __nv_bfloat16* q0, const __nv_bfloat16* q1) {
  const int t = threadIdx.x & 3;
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const int d = kk * 16 + 2 * t;
    qf[kk][0] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
    qf[kk][1] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
    qf[kk][2] = q0 ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
    qf[kk][3] = q1 ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
  }
}

// ---------------------------------------------------------------------------------------
// decode / multi-row verify
//   q          : [B * nq rows][ldq] with head h at column h*128
//   out        : [B * nq][hq][128] bf16
//   part_o     : fp32 [B][nsplit][nq*hq][128], part_ml : fp32 [B][nsplit][nq*hq][2]
//   ctx_lens   : keys visible to the LAST query row of the sequence (includes the nq new tokens)
//   tree_mask  : optional u64 [B][nq]; bit i of row r = key (ctx-nq+i) visible to row r
// grid (nsplit, hkv * row tiles, B), NW warps, each warp owns 64/NW keys of every 64-key page.
// Measured on B200 (batch 64, context 1100, 32/8 heads): four 16-key warps 75.6 us, two 32-key warps
// 80.3 us -- the wider warps issue fewer instructions per key but leave too few warps per SM.
// ---------------------------------------------------------------------------------------
template <int NW>
__global__ void __launch_bounds__(32 * NW)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table,
                   const int* __restrict__ ctx_lens, const unsigned long long* __restrict__ tree_mask,
                   __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml, int hq,
                   int hkv, int nq, int ldq, int max_blocks, int num_blocks, int nsplit, float scale_log2,
                   int* status, int* __restrict__ split_counters, int window, const int* __restrict__ kv_start,
                   int pstride, const float* __restrict__ sinks) {
  pdl_trigger();
  if (threadIdx.x == 0) FF_TL(status, KID_ATTN_DECODE, 0);
  pdl_wait();
  if (threadIdx.x == 0) FF_TL(status, KID_ATTN_DECODE, 1);
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled TMA destinations need 1024-byte alignment
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // blockIdx.y = row tile * hkv + kv head: nq * G packed rows are processed 16 at a time
  const int split = blockIdx.x, kvh = blockIdx.y % hkv, rt = blockIdx.y / hkv, b = blockIdx.z;
  const int G = hq / hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int ctx = ctx_lens[b];
  const int pages = (ctx + PAGE - 1) / PAGE;
  // sliding window (models with local-attention layers; not combined with tree masks): the query at position pos
  // sees keys pos - window + 1 .. pos, so the pages before the earliest bound of the nq queries are not visited
  // kv_start (mixed cache formats): keys below kv_start[b] (a multiple of the page size) are not in BF16 pages any
  // more; another kernel covers them and writes its partials behind this kernel's splits (stride pstride)
  int pfirst = window > 0 ? max(0, ctx - nq - window + 1) / PAGE : 0;
  if (kv_start != nullptr) pfirst = max(pfirst, min(kv_start[b], ctx) / PAGE);
  const int per = (pages - pfirst + nsplit - 1) / nsplit;
  const int p0 = pfirst + split * per, p1 = min(pages, p0 + per);
  const int rows_total = nq * G;
  const int rows_used = min(16, rows_total - rt * 16);

  // rows g and g+8 of the packed tile: packed row r -> (query r / G, head kvh*G + r % G)
  const __nv_bfloat16* qp[2]; int lim[2]; unsigned long long mk[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = rt * 16 + g + e * 8;
    if (r < rows_total) {
      const int qi = r / G, hh = kvh * G + r % G;
      qp[e] = q + (size_t)(b * nq + qi) * ldq + (size_t)hh * HD;
      lim[e] = ctx - nq + qi;
      mk[e] = tree_mask ? tree_mask[(size_t)b * nq + qi] : ~0ull;
    } else { qp[e] = nullptr; lim[e] = -1; mk[e] = 0ull; }
  }
  uint32_t qf[8][4];
  load_q_frags(qf, qp[0], qp[1]);
  RowState st; init_state(st);

  // DEC_STAGES stages of (K page, V page); thread 0 keeps DEC_STAGES-1 pages requested by TMA (four 8-KiB
  // boxes each: K and V, low and high 64 dims) ahead of the page all warps work on
  constexpr int STAGE_BYTES = 2 * PAGE * HD * 2;     // K page + V page
  __shared__ uint64_t full_bar[DEC_STAGES];
  __shared__ int abort_flag;
  bool bad = false;
  // the block ids of this CTA's pages, fetched once by all threads: the page loop then issues its
  // TMA loads without a dependent global load in front of each
  __shared__ int sblk[128];
  for (int i = threadIdx.x; i < 128 && p0 + i < p1; i += 32 * NW) sblk[i] = block_table[(size_t)b * max_blocks + p0 + i];
  if (threadIdx.x == 0) {
    for (int i = 0; i < DEC_STAGES; ++i) mbar_init(&full_bar[i], 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  auto issue = [&](int page_idx, int buf) {
    int blk = (page_idx - p0 < 128) ? sblk[page_idx - p0] : block_table[(size_t)b * max_blocks + page_idx];
    if (blk < 0 || blk >= num_blocks) { bad = true; blk = 0; }
    const int row = (blk * hkv + kvh) * PAGE;
    uint8_t* sk = smem + buf * STAGE_BYTES;
    uint8_t* sv = sk + PAGE * HD * 2;
    mbar_expect_tx(&full_bar[buf], STAGE_BYTES);
    tma_load_2d(sk, &tmK, &full_bar[buf], 0, row);
    tma_load_2d(sk + PAGE * 128, &tmK, &full_bar[buf], 64, row);
    tma_load_2d(sv, &tmV, &full_bar[buf], 0, row);
    tma_load_2d(sv + PAGE * 128, &tmV, &full_bar[buf], 64, row);
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < DEC_STAGES - 1 && p0 + i < p1; ++i) issue(p0 + i, i);
  bool ok = true;
  for (int p = p0; p < p1; ++p) {
    const int it = p - p0, buf = it % DEC_STAGES;
    const uint32_t ph = (it / DEC_STAGES) & 1;
    // the stage refilled here was last read in iteration p-1, which every warp has left (barrier below)
    if (threadIdx.x == 0 && p + DEC_STAGES - 1 < p1) issue(p + DEC_STAGES - 1, (it + DEC_STAGES - 1) % DEC_STAGES);
    if (ok && !mbar_wait(&full_bar[buf], ph, &abort_flag, status, KID_ATTN_DECODE, 1)) ok = false;
    constexpr int KPW = PAGE / NW;                     // keys per warp
    const int key0 = p * PAGE + warp * KPW;
    const uint32_t sk = smem_u32(smem + buf * STAGE_BYTES);
    if (ok && key0 < ctx) {
      bool um = tree_mask != nullptr;
      int ts = ctx - nq;
      unsigned long long a0 = mk[0], a1 = mk[1];
      if (window > 0 && !um) {                         // lower bound of each row as a visibility set over this warp's keys
        const int lo0 = lim[0] - window + 1 - key0, lo1 = lim[1] - window + 1 - key0;
        um = true; ts = key0;
        a0 = lo0 <= 0 ? ~0ull : (lo0 >= 64 ? 0ull : (~0ull << lo0));
        a1 = lo1 <= 0 ? ~0ull : (lo1 >= 64 ? 0ull : (~0ull << lo1));
      }
      warp_tile<KPW / 8>(qf, st, sk, sk + PAGE * HD * 2, warp * KPW, key0, lim[0], lim[1], um, ts, a0, a1, scale_log2);
    }
    __syncthreads();
  }
  if (bad) set_status(status, KID_ATTN_DECODE, FF_ERR_BOUNDS, b, split);

  // merge the four warps through shared memory (reusing the tile buffers)
  float l0 = st.l[0], l1 = st.l[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* so = reinterpret_cast<float*>(smem);              // [NW warps][16 rows][128]
  float* sml = so + NW * 16 * HD;                          // [NW][16][2]
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = i * 8 + 2 * t;
    so[(warp * 16 + g) * HD + d] = st.o[i][0];     so[(warp * 16 + g) * HD + d + 1] = st.o[i][1];
    so[(warp * 16 + g + 8) * HD + d] = st.o[i][2]; so[(warp * 16 + g + 8) * HD + d + 1] = st.o[i][3];
  }
  if (t == 0) {
    sml[(warp * 16 + g) * 2] = st.m[0];     sml[(warp * 16 + g) * 2 + 1] = l0;
    sml[(warp * 16 + g + 8) * 2] = st.m[1]; sml[(warp * 16 + g + 8) * 2 + 1] = l1;
  }
  __syncthreads();
  for (int r = 0; r < rows_used; ++r) {
    const int rg = rt * 16 + r;
    float M = NEG_BIG;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, sml[(w * 16 + r) * 2]);
    float L = 0.f, sc[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) { sc[w] = exp2f(sml[(w * 16 + r) * 2] - M); L += sml[(w * 16 + r) * 2 + 1] * sc[w]; }
    const int qi = rg / G, hh = kvh * G + rg % G;
    for (int d = threadIdx.x; d < HD; d += 32 * NW) {
      float acc = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) acc += so[(w * 16 + r) * HD + d] * sc[w];
      if (nsplit == 1 && pstride == 0) {
        // learnable soft-max: the head's sink logit enters the denominator only
        const float Ls = sinks ? L + exp2f(sinks[hh] * 1.4426950408889634f - M) : L;
        out[((size_t)(b * nq + qi) * hq + hh) * HD + d] = __float2bfloat16(Ls > 0.f ? acc / Ls : 0.f);
      } else {
        const size_t pr = ((size_t)b * (pstride ? pstride : nsplit) + split) * (nq * hq) + (size_t)qi * hq + hh;
        part_o[pr * HD + d] = acc;
        if (d == 0) {
          part_ml[pr * 2] = M; part_ml[pr * 2 + 1] = L;
          dbg_write_once(status, KID_ATTN_DECODE, DBG_ATTN_PARTIAL, (long long)pr);
        }
      }
    }
  }
  if (nsplit > 1 && split_counters != nullptr && pstride == 0) {
    // the split that arrives last merges the partials of this (sequence, kv head, row tile): no second launch
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    const int item = b * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) {
      const int prev = atomicAdd(&split_counters[item], 1);
      s_last = (prev == nsplit - 1);
      if (s_last) split_counters[item] = 0;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int r = 0; r < rows_used; ++r) {
        const int rg = rt * 16 + r, qi = rg / G, hh = kvh * G + rg % G;
        const size_t row = (size_t)qi * hq + hh;
        float M = NEG_BIG;
        for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, __ldcg(&part_ml[(((size_t)b * nsplit + sp) * (nq * hq) + row) * 2]));
        for (int d = threadIdx.x; d < HD; d += 32 * NW) {
          float L = 0.f, acc = 0.f;
          for (int sp = 0; sp < nsplit; ++sp) {
            const size_t pr = ((size_t)b * nsplit + sp) * (nq * hq) + row;
            const float sc = exp2f(__ldcg(&part_ml[pr * 2]) - M);
            L += __ldcg(&part_ml[pr * 2 + 1]) * sc;
            acc += __ldcg(&part_o[pr * HD + d]) * sc;
          }
          if (sinks) L += exp2f(sinks[hh] * 1.4426950408889634f - M);
          out[((size_t)(b * nq + qi) * hq + hh) * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
        }
      }
    }
  }
}

// grid (B * nq * hq), 128 threads
__global__ void __launch_bounds__(128)
attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                  int rows_per_seq, int nsplit, const float* __restrict__ sinks, int hq) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x, b = row / rows_per_seq, r = row % rows_per_seq, d = threadIdx.x;
  float M = NEG_BIG;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(((size_t)b * nsplit + s) * rows_per_seq + r) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const size_t pr = ((size_t)b * nsplit + s) * rows_per_seq + r;
    const float sc = exp2f(part_ml[pr * 2] - M);
    L += part_ml[pr * 2 + 1] * sc;
    acc += part_o[pr * HD + d] * sc;
  }
  if (sinks) L += exp2f(sinks[r % hq] * 1.4426950408889634f - M);
  out[(size_t)row * HD + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
}

// ---------------------------------------------------------------------------------------
// prefill (causal, chunked): sequence b owns query rows [q_start[b], q_start[b] + q_len[b]) of
// the packed buffer and ctx_lens[b] keys in the cache (past + this chunk). Query i sits at
// position ctx - q_len + i. grid (ceil(max_q_len/64), hq, B), 128 threads.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kcache,
                    const __nv_bfloat16* __restrict__ vcache, const int* __restrict__ block_table,
                    const int* __restrict__ q_start, const int* __restrict__ q_lens, const int* __restrict__ ctx_lens,
                    __nv_bfloat16* __restrict__ out, int hq, int hkv, int ldq, int ldo, int max_blocks, int num_blocks,
                    float scale_log2, int window, int causal, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int b = blockIdx.z, h = blockIdx.y;
  const int qlen = q_lens[b];
  const int tile0 = blockIdx.x * 64;
  if (tile0 >= qlen) return;
  const int ctx = ctx_lens[b], qs = q_start[b];
  const int kvh = h / (hq / hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int past = ctx - qlen;
  const __nv_bfloat16* qp[2]; int lim[2]; int rowi[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int i = tile0 + warp * 16 + g + e * 8;
    rowi[e] = i;
    if (i < qlen) { qp[e] = q + (size_t)(qs + i) * ldq + (size_t)h * HD; lim[e] = causal ? past + i : ctx - 1; }
    else { qp[e] = nullptr; lim[e] = -1; }
  }
  uint32_t qf[8][4];
  load_q_frags(qf, qp[0], qp[1]);
  RowState st; init_state(st);
  const int last_key = causal ? past + min(qlen, tile0 + 64) - 1 : ctx - 1;   // bidirectional: every key
  int first_key = 0;
  if (window > 0) first_key = max(0, past + tile0 - window + 1);
  const int p0 = first_key / PAGE, p1 = last_key / PAGE + 1;
  const int warp_last = causal ? past + min(qlen - 1, tile0 + warp * 16 + 15) : ctx - 1;

  uint8_t* sKbuf[2] = {smem, smem + 2 * PAGE * HD * 2};
  uint8_t* sVbuf[2] = {smem + PAGE * HD * 2, smem + 3 * PAGE * HD * 2};
  bool bad = false;
  auto issue = [&](int page_idx, int buf) {
    int blk = block_table[(size_t)b * max_blocks + page_idx];
    if (blk < 0 || blk >= num_blocks) { bad = true; blk = 0; }
    const size_t base = ((size_t)blk * hkv + kvh) * PAGE * HD;
    load_tile_async(sKbuf[buf], kcache + base, PAGE, threadIdx.x, 128);
    load_tile_async(sVbuf[buf], vcache + base, PAGE, threadIdx.x, 128);
    cp_async_commit();
  };
  issue(p0, 0);
  for (int p = p0; p < p1; ++p) {
    const int buf = (p - p0) & 1;
    if (p + 1 < p1) { issue(p + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    if (p * PAGE <= warp_last) {
      int l0 = lim[0], l1 = lim[1];
      // sliding window: a row at position pos sees keys pos - window + 1 .. pos. Whole pages before the tile's
      // earliest bound are skipped (first_key); inside a page the lower bound goes through the per-row 64-bit
      // visibility set of the tile routine (bit i = key page_start + i visible).
      unsigned long long m0 = ~0ull, m1 = ~0ull;
      if (window > 0) {
        const int lo0 = l0 - window + 1 - p * PAGE, lo1 = l1 - window + 1 - p * PAGE;
        m0 = lo0 <= 0 ? ~0ull : (lo0 >= 64 ? 0ull : (~0ull << lo0));
        m1 = lo1 <= 0 ? ~0ull : (lo1 >= 64 ? 0ull : (~0ull << lo1));
      }
      warp_tile<8>(qf, st, smem_u32(sKbuf[buf]), smem_u32(sVbuf[buf]), 0, p * PAGE, l0, l1, window > 0, p * PAGE, m0, m1,
                   scale_log2);
    }
    __syncthreads();
  }
  if (bad) set_status(status, KID_ATTN_PREFILL, FF_ERR_BOUNDS, b, blockIdx.x);
  float l0 = st.l[0], l1 = st.l[1];
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int d = i * 8 + 2 * t;
    if (rowi[0] < qlen)
      *reinterpret_cast<uint32_t*>(out + (size_t)(qs + rowi[0]) * ldo + (size_t)h * HD + d) =
          pack_bf16x2(st.o[i][0] * i0, st.o[i][1] * i0);
    if (rowi[1] < qlen)
      *reinterpret_cast<uint32_t*>(out + (size_t)(qs + rowi[1]) * ldo + (size_t)h * HD + d) =
          pack_bf16x2(st.o[i][2] * i1, st.o[i][3] * i1);
  }
}

}  // namespace ff
using namespace ff;

constexpr int ATTN_SMEM = 4 * PAGE * HD * 2;   // 64 KiB: two stages of K and V pages (prefill)
constexpr int DEC_SMEM = DEC_STAGES * 2 * PAGE * HD * 2 + 1024;

// Waves of CTAs the split-KV plan aims for (calibrated; default four).
static int g_attn_waves = 4;
FF_EXPORT int ff_attn_decode_set_waves(int waves) {
  if (waves < 1 || waves > 16) return FF_HOST_BAD_SHAPE;
  g_attn_waves = waves;
  return 0;
}

// Number of KV splits the decode launcher will use and the scratch it needs.
FF_EXPORT int ff_attn_decode_plan(int batch, int hq, int hkv, int nq, int max_ctx, long long* part_o_bytes,
                                  long long* part_ml_bytes) {
  const int pages = (max_ctx + PAGE - 1) / PAGE;
  const int ctas = batch * hkv * ((nq * (hq / hkv) + 15) / 16);
  int nsplit = 1;
  // three 64-KiB CTAs fit on one SM; aim for at least four full waves so the ragged last wave
  // costs little
  const int target = 148 * 3 * g_attn_waves;
  if (ctas < target) nsplit = (target + ctas - 1) / ctas;
  if (const char* ev = getenv("FF_ATTN_NSPLIT")) { const int v = atoi(ev); if (v > 0) nsplit = v; }
  if (nsplit > pages) nsplit = pages;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 64) nsplit = 64;
  if (part_o_bytes) *part_o_bytes = (long long)batch * nsplit * nq * hq * HD * 4;
  if (part_ml_bytes) *part_ml_bytes = (long long)batch * nsplit * nq * hq * 2 * 4;
  return nsplit;
}

static int attn_decode_launch(const void* q, const void* kcache, const void* vcache, const int* block_table,
                              const int* ctx_lens, const unsigned long long* tree_mask, void* out, float* part_o,
                              float* part_ml, int batch, int hq, int hkv, int head_dim, int nq, int ldq, int max_blocks,
                              int num_blocks, int nsplit, float scale, int* split_counters, int* status, cudaStream_t s,
                              int window, const int* kv_start = nullptr, int pstride = 0, const float* sinks = nullptr) {
  if (window > 0 && tree_mask) return FF_HOST_UNSUPPORTED;
  if (pstride != 0 && (pstride < nsplit || !part_o || !part_ml)) return FF_HOST_BAD_SHAPE;
  if (head_dim != HD || batch <= 0 || hq <= 0 || hkv <= 0 || hq % hkv) return FF_HOST_BAD_SHAPE;
  if (nq < 1 || nq > 64) return FF_HOST_BAD_SHAPE;
  if (ldq % 8 || nsplit < 1) return FF_HOST_BAD_ALIGN;
  if (nsplit > 1 && (!part_o || !part_ml)) return FF_HOST_BAD_SHAPE;
  constexpr int NW = DEC_WARPS;
  if (int r = opt_in_smem(attn_decode_kernel<NW>, DEC_SMEM)) return r;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int row_tiles = (nq * (hq / hkv) + 15) / 16;
  dim3 grid(nsplit, hkv * row_tiles, batch);
  // the caches as [blocks * hkv * 64 rows][128]; a box is one half (64 dims) of one page of one head
  CUtensorMap tmK, tmV;
  const uint64_t cache_rows = (uint64_t)num_blocks * hkv * PAGE;
  if (int r = make_tmap_2d(&tmK, kcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, HD, cache_rows, HD * 2, 64, PAGE)) return r;
  if (int r = make_tmap_2d(&tmV, vcache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, HD, cache_rows, HD * 2, 64, PAGE)) return r;
  if (int lr_ = launch_pdl(attn_decode_kernel<NW>, dim3(grid), dim3(32 * NW), DEC_SMEM, s, 0, tmK, tmV, (const __nv_bfloat16*)q,
      block_table, ctx_lens, tree_mask, (__nv_bfloat16*)out, part_o, part_ml, hq, hkv, nq,
      ldq, max_blocks, num_blocks, nsplit, scale_log2, status, split_counters, window, kv_start, pstride, sinks)) return lr_;
  if (int r = launch_result()) return r;
  if (pstride != 0) return 0;                      // partials only: the caller merges after the other kernel has added its own
  if (nsplit > 1 && split_counters == nullptr) {
    if (int lr_ = launch_pdl(attn_merge_kernel, dim3(batch * nq * hq), dim3(128), 0, s, 0, part_o, part_ml, (__nv_bfloat16*)out, nq * hq, nsplit, sinks, hq)) return lr_;
    return launch_result();
  }
  return 0;
}

FF_EXPORT int ff_attn_decode(const void* q, const void* kcache, const void* vcache, const int* block_table,
                             const int* ctx_lens, const unsigned long long* tree_mask, void* out, float* part_o,
                             float* part_ml, int batch, int hq, int hkv, int head_dim, int nq, int ldq, int max_blocks,
                             int num_blocks, int nsplit, float scale, int* split_counters, int* status, cudaStream_t s) {
  return attn_decode_launch(q, kcache, vcache, block_table, ctx_lens, tree_mask, out, part_o, part_ml, batch, hq, hkv,
                            head_dim, nq, ldq, max_blocks, num_blocks, nsplit, scale, split_counters, status, s, 0);
}

// BF16 part of a decode step over a cache whose older keys are sealed in the 8-bit store: visits the pages from
// kv_start[b] on and writes partials only, at split indices [0, nsplit) of a buffer with `pstride` splits per
// sequence; ff_attn_merge finishes after the sealed-part kernel has written the other splits.
FF_EXPORT int ff_attn_decode_partial(const void* q, const void* kcache, const void* vcache, const int* block_table,
                                     const int* ctx_lens, const int* kv_start, float* part_o, float* part_ml, int batch,
                                     int hq, int hkv, int head_dim, int ldq, int max_blocks, int num_blocks, int nsplit,
                                     int pstride, float scale, int* status, cudaStream_t s) {
  if (!kv_start || pstride < 1) return FF_HOST_BAD_SHAPE;
  return attn_decode_launch(q, kcache, vcache, block_table, ctx_lens, nullptr, nullptr, part_o, part_ml, batch, hq, hkv,
                            head_dim, 1, ldq, max_blocks, num_blocks, nsplit, scale, nullptr, status, s, 0, kv_start, pstride);
}

// Merge `nsplit` partials per (sequence row, head) into out [rows * hq, 128] bf16.
FF_EXPORT int ff_attn_merge(const float* part_o, const float* part_ml, void* out, int batch, int rows_per_seq, int nsplit,
                            cudaStream_t s) {
  if (batch <= 0 || rows_per_seq <= 0 || nsplit < 1) return FF_HOST_BAD_SHAPE;
  if (int lr_ = launch_pdl(attn_merge_kernel, dim3(batch * rows_per_seq), dim3(128), 0, s, 0, part_o, part_ml,
                           (__nv_bfloat16*)out, rows_per_seq, nsplit, (const float*)nullptr, rows_per_seq)) return lr_;
  return launch_result();
}

// Decode attention with a learnable soft-max (one sink logit per query head in the denominator, sinks: float[hq]) and an
// optional sliding window (window = 0: full attention). No tree mask.
FF_EXPORT int ff_attn_decode_sink(const void* q, const void* kcache, const void* vcache, const int* block_table,
                                  const int* ctx_lens, void* out, float* part_o, float* part_ml, int batch, int hq,
                                  int hkv, int head_dim, int nq, int ldq, int max_blocks, int num_blocks, int nsplit,
                                  float scale, int window, const float* sinks, int* status, cudaStream_t s) {
  if (window < 0 || sinks == nullptr) return FF_HOST_BAD_SHAPE;
  return attn_decode_launch(q, kcache, vcache, block_table, ctx_lens, nullptr, out, part_o, part_ml, batch, hq, hkv,
                            head_dim, nq, ldq, max_blocks, num_blocks, nsplit, scale, nullptr, status, s, window, nullptr, 0,
                            sinks);
}

// Decode attention of a local-attention layer: every query sees its last `window` keys.
FF_EXPORT int ff_attn_decode_window(const void* q, const void* kcache, const void* vcache, const int* block_table,
                                    const int* ctx_lens, void* out, float* part_o, float* part_ml, int batch, int hq,
                                    int hkv, int head_dim, int nq, int ldq, int max_blocks, int num_blocks, int nsplit,
                                    float scale, int window, int* split_counters, int* status, cudaStream_t s) {
  if (window <= 0) return FF_HOST_BAD_SHAPE;
  return attn_decode_launch(q, kcache, vcache, block_table, ctx_lens, nullptr, out, part_o, part_ml, batch, hq, hkv,
                            head_dim, nq, ldq, max_blocks, num_blocks, nsplit, scale, split_counters, status, s, window);
}

// window > 0: sliding window (exact); 0: causal; < 0: bidirectional (every query sees all ctx keys:
// encoder / vision-tower attention over a segment stored in the paged layout).
FF_EXPORT int ff_attn_prefill(const void* q, const void* kcache, const void* vcache, const int* block_table,
                              const int* q_start, const int* q_lens, const int* ctx_lens, void* out, int batch,
                              int max_q_len, int hq, int hkv, int head_dim, int ldq, int ldo, int max_blocks,
                              int num_blocks, float scale, int window, int* status, cudaStream_t s) {
  if (head_dim != HD || batch <= 0 || max_q_len <= 0 || hq % hkv) return FF_HOST_BAD_SHAPE;
  if (ldq % 8 || ldo % 2) return FF_HOST_BAD_ALIGN;
  if (int r = opt_in_smem(attn_prefill_kernel, ATTN_SMEM)) return r;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((max_q_len + 63) / 64, hq, batch);
  attn_prefill_kernel<<<grid, 128, ATTN_SMEM, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kcache,
      (const __nv_bfloat16*)vcache, block_table, q_start, q_lens, ctx_lens, (__nv_bfloat16*)out, hq, hkv, ldq, ldo,
      max_blocks, num_blocks, scale_log2, window < 0 ? 0 : window, window < 0 ? 0 : 1, status);
  return launch_result();
}
