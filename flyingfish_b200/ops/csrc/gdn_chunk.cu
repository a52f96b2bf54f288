// Gated delta rule, chunked prefill form on tensor cores (head dims 128 x 128, chunks of 64 tokens).
//
// The recurrence   S <- e^{g_t} S ;  d_t = beta_t (v_t - S^T k_t) ;  S <- S + k_t d_t^T ;  o_t = S^T q_t
// over a chunk with cumulative log-decay c_t = g_1 + .. + g_t and incoming state S0 is, in matrix form
//     A[t,i] = beta_t e^{c_t - c_i} (k_t . k_i)   (i < t),     T = (I + A)^-1                       (WY representation)
//     W = T (beta e^{c} K)        U = T (beta V)       D = U - W S0                                  (the deltas d_t)
//     O = (e^{c} Q) S0 + (M . Q K^T) D,   M[t,i] = e^{c_t - c_i} (i <= t)
//     S <- e^{c_C} S0 + (e^{c_C - c} K)^T D
// Seven small matrix products per chunk run as mma.sync m16n8k16 (BF16 operands, FP32 accumulation) out of shared
// memory tiles; the triangular inverse is a forward substitution with four lanes per column. The state lives in the
// accumulator registers of the last product for the whole sequence (FP32) and is mirrored to shared memory in BF16
// once per chunk as the operand of the products that read it. One CTA (256 threads) per (sequence, head) walks the
// chunks in order. The reference's chunk-wise kernels are kernels/gdn/gdn_chunkwise_p1.cu and gdn_cw_p2.cu (two
// passes: the S-independent part of all chunks in parallel, then the sequential pass); this kernel does both per chunk.
#include "ptx.cuh"
#include "host_util.h"
#include "mma_sync.cuh"

namespace ff {

constexpr int GC = 64;       // tokens per chunk
constexpr int GD = 128;      // key and value dims
constexpr int GCH = GD / 8;  // 16-byte chunks per 128-wide row

struct GdnSmem {
  uint8_t q[GC * GD * 2];        // Q, later e^{c} Q
  uint8_t k[GC * GD * 2];        // K, later e^{c_C - c} K
  uint8_t v[GC * GD * 2];        // V
  uint8_t w[GC * GD * 2];        // -W
  uint8_t d[GC * GD * 2];        // D
  uint8_t s16[GD * GD * 2];      // state mirror [k dim][v dim]
  float a[GC * GC];              // A (strictly lower)
  uint8_t t1[GC * GC * 2];       // T with columns scaled by beta e^{c}
  uint8_t t2[GC * GC * 2];       // T with columns scaled by beta
  uint8_t p[GC * GC * 2];        // M . Q K^T
  float beta[GC], c[GC], ec[GC], bec[GC], edec[GC];   // beta, c_t, e^{c_t}, beta e^{c_t}, e^{c_C - c_t}
};

// store a pair of accumulator values as BF16 at (row, col .. col+1) of a swizzled tile with `chunks` 16-byte chunks per row
__device__ __forceinline__ void gdn_store2(uint8_t* tile, int row, int col, int chunks, float x, float y) {
  *reinterpret_cast<uint32_t*>(tile + ms_off(row, col >> 3, chunks) + (col & 7) * 2) = pack_bf16x2(x, y);
}

// acc[NT][4] (+)= A[m0 .. m0+15][0 .. 16 KS) . B, A row-major tile (a_chunks per row);
// B_TRANS = false: B given as [n][k] rows (b_chunks per row), n-tiles n0 .. n0 + 8 NT
// B_TRANS = true : B given as [k][n] rows, same n range
template <int NT, int KS, bool B_TRANS>
__device__ __forceinline__ void gdn_mma(float (&acc)[NT][4], uint32_t a_base, int a_chunks, int m0, uint32_t b_base, int b_chunks,
                                        int n0, int lane) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    uint32_t a[4];
    ms_ldsm4(a_base + ms_off(m0 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * ks + (lane >> 4), a_chunks), a[0], a[1], a[2], a[3]);
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b0, b1, b2, b3;
      if (B_TRANS) {
        const int krow = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        ms_ldsm4t(b_base + ms_off(krow, (n0 >> 3) + 2 * np + (lane >> 4), b_chunks), b0, b1, b2, b3);
      } else {
        ms_ldsm4(b_base + ms_off(n0 + 16 * np + ((lane >> 4) << 3) + (lane & 7), 2 * ks + ((lane >> 3) & 1), b_chunks), b0, b1, b2, b3);
      }
      ms_mma(acc[2 * np], a, b0, b1);
      ms_mma(acc[2 * np + 1], a, b2, b3);
    }
  }
}

// grid (heads, sequences), 256 threads. q, k, v [rows, heads, 128] f32; beta, g [rows, heads] f32;
// S [slots, heads, 128, 128] f32 (read at the start, written at the end); out [rows, heads, 128] bf16.
__global__ void __launch_bounds__(256, 1)
gdn_chunked_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ beta, const float* __restrict__ g, float* __restrict__ S,
                   __nv_bfloat16* __restrict__ out, const int* __restrict__ row_start, const int* __restrict__ state_slot,
                   int heads) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t gdn_raw[];
  GdnSmem& sm = *reinterpret_cast<GdnSmem*>((reinterpret_cast<uintptr_t>(gdn_raw) + 127) & ~uintptr_t(127));
  const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int r0 = row_start[seq], r1 = row_start[seq + 1];
  if (r1 <= r0) return;
  const int slot = state_slot ? state_slot[seq] : seq;
  float* Sg = S + ((size_t)slot * heads + h) * GD * GD;
  const uint32_t aQ = smem_u32(sm.q), aK = smem_u32(sm.k), aV = smem_u32(sm.v), aW = smem_u32(sm.w), aD = smem_u32(sm.d),
                 aS = smem_u32(sm.s16), aT1 = smem_u32(sm.t1), aT2 = smem_u32(sm.t2), aP = smem_u32(sm.p);

  // state: warp w holds rows (key dims) 16w .. 16w+15, all 128 value dims, as accumulator fragments
  float st[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int col = nt * 8 + 2 * tq;
    const float2 lo = *reinterpret_cast<const float2*>(Sg + (size_t)(warp * 16 + gq) * GD + col);
    const float2 hi = *reinterpret_cast<const float2*>(Sg + (size_t)(warp * 16 + gq + 8) * GD + col);
    st[nt][0] = lo.x; st[nt][1] = lo.y; st[nt][2] = hi.x; st[nt][3] = hi.y;
  }

  for (int c0 = r0; c0 < r1; c0 += GC) {
    const int n = min(GC, r1 - c0);
    __syncthreads();                                   // the previous chunk's tiles are no longer read
    // ---- load the chunk: Q, K, V as BF16 tiles (rows beyond n are zero), beta, cumulative decay
    for (int i = tid; i < GC * GCH; i += 256) {
      const int t = i / GCH, cch = i - t * GCH;
      uint4 qv = make_uint4(0, 0, 0, 0), kv = qv, vv = qv;
      if (t < n) {
        const size_t base = ((size_t)(c0 + t) * heads + h) * GD + cch * 8;
        const float4 q0 = *reinterpret_cast<const float4*>(q + base), q1 = *reinterpret_cast<const float4*>(q + base + 4);
        const float4 k0 = *reinterpret_cast<const float4*>(k + base), k1 = *reinterpret_cast<const float4*>(k + base + 4);
        const float4 v0 = *reinterpret_cast<const float4*>(v + base), v1 = *reinterpret_cast<const float4*>(v + base + 4);
        qv = make_uint4(pack_bf16x2(q0.x, q0.y), pack_bf16x2(q0.z, q0.w), pack_bf16x2(q1.x, q1.y), pack_bf16x2(q1.z, q1.w));
        kv = make_uint4(pack_bf16x2(k0.x, k0.y), pack_bf16x2(k0.z, k0.w), pack_bf16x2(k1.x, k1.y), pack_bf16x2(k1.z, k1.w));
        vv = make_uint4(pack_bf16x2(v0.x, v0.y), pack_bf16x2(v0.z, v0.w), pack_bf16x2(v1.x, v1.y), pack_bf16x2(v1.z, v1.w));
      }
      *reinterpret_cast<uint4*>(sm.q + ms_off(t, cch, GCH)) = qv;
      *reinterpret_cast<uint4*>(sm.k + ms_off(t, cch, GCH)) = kv;
      *reinterpret_cast<uint4*>(sm.v + ms_off(t, cch, GCH)) = vv;
    }
    if (warp == 0) {
      // inclusive scan of g over the chunk (two elements per lane); padded tokens have g = 0, beta = 0
      const int t0 = 2 * lane, t1 = 2 * lane + 1;
      const float g0 = t0 < n ? g[(size_t)(c0 + t0) * heads + h] : 0.f;
      const float g1 = t1 < n ? g[(size_t)(c0 + t1) * heads + h] : 0.f;
      float run = g0 + g1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const float up = __shfl_up_sync(0xffffffffu, run, o); if (lane >= o) run += up; }
      const float c1 = run, cc0 = run - g1;
      const float total = __shfl_sync(0xffffffffu, run, 31);
      const float b0 = t0 < n ? beta[(size_t)(c0 + t0) * heads + h] : 0.f;
      const float b1 = t1 < n ? beta[(size_t)(c0 + t1) * heads + h] : 0.f;
      sm.c[t0] = cc0; sm.c[t1] = c1;
      sm.beta[t0] = b0; sm.beta[t1] = b1;
      sm.ec[t0] = __expf(cc0); sm.ec[t1] = __expf(c1);
      sm.bec[t0] = b0 * __expf(cc0); sm.bec[t1] = b1 * __expf(c1);
      sm.edec[t0] = __expf(total - cc0); sm.edec[t1] = __expf(total - c1);
    }
    // state mirror in BF16 [k dim][v dim]
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      gdn_store2(sm.s16, warp * 16 + gq, nt * 8 + 2 * tq, GCH, st[nt][0], st[nt][1]);
      gdn_store2(sm.s16, warp * 16 + gq + 8, nt * 8 + 2 * tq, GCH, st[nt][2], st[nt][3]);
    }
    __syncthreads();

    // ---- K K^T and Q K^T (64 x 64 each): warp w -> rows 16 (w & 3), columns 32 (w >> 2) .. + 31
    {
      const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;
      float kk[4][4], qk[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { kk[i][0] = kk[i][1] = kk[i][2] = kk[i][3] = 0.f; qk[i][0] = qk[i][1] = qk[i][2] = qk[i][3] = 0.f; }
      gdn_mma<4, GD / 16, false>(kk, aK, GCH, m0, aK, GCH, n0, lane);
      gdn_mma<4, GD / 16, false>(qk, aQ, GCH, m0, aK, GCH, n0, lane);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int t = m0 + gq + 8 * e;
          const float ct = sm.c[t], bt = sm.beta[t];
          float pa[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int i = n0 + nt * 8 + 2 * tq + j;
            const float dec = (i <= t) ? __expf(ct - sm.c[i]) : 0.f;
            sm.a[t * GC + i] = (i < t) ? bt * dec * kk[nt][2 * e + j] : 0.f;
            pa[j] = dec * qk[nt][2 * e + j];
          }
          gdn_store2(sm.p, t, n0 + nt * 8 + 2 * tq, GC / 8, pa[0], pa[1]);
        }
    }
    __syncthreads();

    // ---- T = (I + A)^-1 by forward substitution: column j on lanes 4j .. 4j+3, lane p keeps T[i][j] for i = p mod 4
    {
      const int j = tid >> 2, p = tid & 3;
      float colp[GC / 4];
#pragma unroll
      for (int i = 0; i < GC / 4; ++i) colp[i] = 0.f;
#pragma unroll
      for (int t = 0; t < GC; ++t) {
        float part = 0.f;
#pragma unroll
        for (int ii = 0; ii < GC / 4; ++ii)
          if (4 * ii < t) {                              // rows 4 ii + p < t contribute (the entries at or past t are still zero)
            const int i = 4 * ii + p;
            part += (i < t) ? sm.a[t * GC + i] * colp[ii] : 0.f;
          }
        part += __shfl_xor_sync(0xffffffffu, part, 1);
        part += __shfl_xor_sync(0xffffffffu, part, 2);
        const float val = (t == j ? 1.f : 0.f) - part;
        if (p == (t & 3)) colp[t >> 2] = val;
      }
      // T[i][j] with the column scaled: t1 by beta_j e^{c_j} (for W), t2 by beta_j (for U)
      const float s1 = sm.bec[j], s2 = sm.beta[j];
#pragma unroll
      for (int ii = 0; ii < GC / 4; ++ii) {
        const int i = 4 * ii + p;
        const float tv = colp[ii];
        *reinterpret_cast<__nv_bfloat16*>(sm.t1 + ms_off(i, j >> 3, GC / 8) + (j & 7) * 2) = __float2bfloat16(tv * s1);
        *reinterpret_cast<__nv_bfloat16*>(sm.t2 + ms_off(i, j >> 3, GC / 8) + (j & 7) * 2) = __float2bfloat16(tv * s2);
      }
    }
    __syncthreads();

    // ---- 64 x 128 products: warp w -> rows 16 (w & 3), columns 64 (w >> 2) .. + 63
    const int m0 = (warp & 3) * 16, n0 = (warp >> 2) * 64;
    {
      float wacc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) wacc[i][0] = wacc[i][1] = wacc[i][2] = wacc[i][3] = 0.f;
      gdn_mma<8, GC / 16, true>(wacc, aT1, GC / 8, m0, aK, GCH, n0, lane);           // W = T1 K
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        gdn_store2(sm.w, m0 + gq, n0 + nt * 8 + 2 * tq, GCH, -wacc[nt][0], -wacc[nt][1]);
        gdn_store2(sm.w, m0 + gq + 8, n0 + nt * 8 + 2 * tq, GCH, -wacc[nt][2], -wacc[nt][3]);
      }
    }
    float dacc[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) dacc[i][0] = dacc[i][1] = dacc[i][2] = dacc[i][3] = 0.f;
    gdn_mma<8, GC / 16, true>(dacc, aT2, GC / 8, m0, aV, GCH, n0, lane);             // U = T2 V
    __syncthreads();                                                                  // -W complete; K no longer read raw
    gdn_mma<8, GD / 16, true>(dacc, aW, GCH, m0, aS, GCH, n0, lane);                 // D = U - W S0
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
      gdn_store2(sm.d, m0 + gq, n0 + nt * 8 + 2 * tq, GCH, dacc[nt][0], dacc[nt][1]);
      gdn_store2(sm.d, m0 + gq + 8, n0 + nt * 8 + 2 * tq, GCH, dacc[nt][2], dacc[nt][3]);
    }
    // scale Q rows by e^{c_t} and K rows by e^{c_C - c_t} in place (each thread its own elements; both tiles were last
    // read before the barrier above)
    for (int i = tid; i < GC * GCH; i += 256) {
      const int t = i / GCH, cch = i - t * GCH;
      const float sq = sm.ec[t], sk = sm.edec[t];
      uint4* qp = reinterpret_cast<uint4*>(sm.q + ms_off(t, cch, GCH));
      uint4* kp = reinterpret_cast<uint4*>(sm.k + ms_off(t, cch, GCH));
      uint4 qv = *qp, kv = *kp;
      uint32_t* qw = reinterpret_cast<uint32_t*>(&qv);
      uint32_t* kw = reinterpret_cast<uint32_t*>(&kv);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 a = unpack_bf16x2(qw[u]), b = unpack_bf16x2(kw[u]);
        qw[u] = pack_bf16x2(a.x * sq, a.y * sq);
        kw[u] = pack_bf16x2(b.x * sk, b.y * sk);
      }
      *qp = qv; *kp = kv;
    }
    __syncthreads();

    // ---- O = (e^{c} Q) S0 + P D
    {
      float oacc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
      gdn_mma<8, GD / 16, true>(oacc, aQ, GCH, m0, aS, GCH, n0, lane);
      gdn_mma<8, GC / 16, true>(oacc, aP, GC / 8, m0, aD, GCH, n0, lane);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = m0 + gq + 8 * e;
        if (t < n) {
          __nv_bfloat16* orow = out + ((size_t)(c0 + t) * heads + h) * GD;
#pragma unroll
          for (int nt = 0; nt < 8; ++nt)
            *reinterpret_cast<uint32_t*>(orow + n0 + nt * 8 + 2 * tq) = pack_bf16x2(oacc[nt][2 * e], oacc[nt][2 * e + 1]);
        }
      }
    }
    // ---- S <- e^{c_C} S0 + (e^{c_C - c} K)^T D : warp w -> key dims 16 w .. 16 w + 15; A operand read transposed from the K tile
    {
      const float total = sm.edec[0] * sm.ec[0];           // e^{c_C}
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) { st[nt][0] *= total; st[nt][1] *= total; st[nt][2] *= total; st[nt][3] *= total; }
#pragma unroll
      for (int ks = 0; ks < GC / 16; ++ks) {
        uint32_t a[4];
        // A[m = key dim][k = token] from K stored [token][key dim]: transposed 8x8 loads
        ms_ldsm4t(aK + ms_off(ks * 16 + (lane & 7) + ((lane >> 4) << 3), warp * 2 + ((lane >> 3) & 1), GCH), a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int np = 0; np < 8; ++np) {
          uint32_t b0, b1, b2, b3;
          const int krow = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          ms_ldsm4t(aD + ms_off(krow, 2 * np + (lane >> 4), GCH), b0, b1, b2, b3);
          ms_mma(st[2 * np], a, b0, b1);
          ms_mma(st[2 * np + 1], a, b2, b3);
        }
      }
    }
  }
  // final state back to global memory
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    const int col = nt * 8 + 2 * tq;
    *reinterpret_cast<float2*>(Sg + (size_t)(warp * 16 + gq) * GD + col) = make_float2(st[nt][0], st[nt][1]);
    *reinterpret_cast<float2*>(Sg + (size_t)(warp * 16 + gq + 8) * GD + col) = make_float2(st[nt][2], st[nt][3]);
  }
}

}  // namespace ff
using namespace ff;

// Chunked prefill form of ff_gdn_recurrent_slots (same arguments, same result up to BF16 operand rounding of the
// matrix products). state_slot may be null (sequence s uses state s).
FF_EXPORT int ff_gdn_chunked_slots(const float* q, const float* k, const float* v, const float* beta, const float* g,
                                   float* S, void* out, const int* row_start, const int* state_slot, int sequences,
                                   int heads, cudaStream_t s) {
  if (sequences <= 0 || heads <= 0) return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(S) & 7)) return FF_HOST_BAD_ALIGN;
  const int smem = (int)sizeof(GdnSmem) + 128;
  if (int r = opt_in_smem(gdn_chunked_kernel, smem)) return r;
  if (int lr = launch_pdl(gdn_chunked_kernel, dim3(heads, sequences), dim3(256), smem, s, 0, q, k, v, beta, g, S,
                          (__nv_bfloat16*)out, row_start, state_slot, heads)) return lr;
  return launch_result();
}
