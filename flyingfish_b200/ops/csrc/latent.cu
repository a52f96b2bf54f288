// Latent window attention (DeepSeek-V4.1-style mixer): decode over a per-sequence ring of FP8 latent
// K rows with one attention sink per head.
//
//   * ring: post-RoPE K rows quantised to E4M3 over the whole head vector, one E8M0 scale per 32
//     codes (amax floored at 1e-4, scale = 2^ceil(log2(amax / 448))); row of position p lives in
//     slot p % window of its sequence's ring.
//   * one KV head shared by all query heads; the value IS the K content (latent attention).
//   * visible keys = the ring, oldest first, minus slots not written yet; score scale given by the
//     caller (head_dim^-0.5).
//   * blocked soft-max in 64-key blocks: every block rescales the FP32 accumulator and the running
//     sum by exp(m_prev - m_new), rounds P to BF16 against the running maximum and adds its
//     UNROUNDED sum; the per-head sink is one extra logit that enters only the denominator, after
//     the last block; one divide; the result is rounded to BF16.
//   * the last rope_tail dims of the output get the inverse rotary (adjacent pairs), then BF16.
// This restates the reference's kernels/latent_window_attention.cu (:1-30 contract, :51-275 core,
// :307-348 ring write / activation quantisation) for batches of sequences: the reference runs one
// block per head with scalar or per-key mma code for a single sequence; here a CTA owns 16 heads of one
// sequence, de-quantises a 64-key block once into shared memory and does Q·Kᵀ and P·V with
// mma.sync m16n8k16 (heads are the M dimension since all heads share the keys).
#include "ptx.cuh"
#include "host_util.h"
#include <cuda_fp8.h>

namespace ff {

constexpr int LW_KEYS = 64;        // keys per soft-max block
constexpr int LW_MAXD = 512;

__device__ __forceinline__ float lw_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float lw_e8m0(uint8_t c) { return __uint_as_float(c == 0 ? 0x00400000u : ((uint32_t)c << 23)); }
__device__ __forceinline__ void lw_ldsm4(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lw_ldsm4t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lw_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// [rows][D] bf16 tile, 16-byte chunk index XORed with row % 8 in its low three bits
__device__ __forceinline__ uint32_t lw_off(int r, int c, int chunks) { return (uint32_t)((r * chunks + ((c & ~7) | ((c ^ r) & 7))) * 16); }

// One warp per 32-element group: codes + E8M0 scale. ring_ids/positions null -> linear layout
// (codes [rows, D], scales [rows, D/32]); else row r goes to slot positions[r] % window of ring ring_ids[r].
__global__ void latent_quant_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ codes,
                                    uint8_t* __restrict__ scales, const int* __restrict__ ring_ids,
                                    const int* __restrict__ positions, long long rows, int D, int ldx, int window,
                                    int rings, int* status) {
  pdl_trigger();
  pdl_wait();
  const int groups = D / 32;
  const long long warp = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (warp >= rows * groups) return;
  const int lane = threadIdx.x & 31;
  const long long row = warp / groups; const int grp = (int)(warp - row * groups);
  const float v = __bfloat162float(x[row * ldx + grp * 32 + lane]);
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  amax = fmaxf(amax, 1e-4f);
  // exponent = ceil(log2(amax / 448))
  const float ratio = amax * (1.0f / 448.0f);
  int ex; const float mant = frexpf(ratio, &ex);            // ratio = mant * 2^ex, mant in [0.5, 1)
  const int exponent = (mant == 0.5f) ? ex - 1 : ex;
  const float scale = ldexpf(1.0f, exponent);
  const uint8_t code = (uint8_t)__nv_cvt_float_to_fp8(fminf(448.f, fmaxf(-448.f, v / scale)), __NV_SATFINITE, __NV_E4M3);
  long long drow = row;
  if (ring_ids != nullptr) {
    const int ring = ring_ids[row], pos = positions[row];
    if (ring < 0 || ring >= rings || pos < 0) { if (lane == 0) set_status(status, KID_LATENT, FF_ERR_BOUNDS, (int)row, ring); return; }
    drow = (long long)ring * window + pos % window;
  }
  codes[drow * D + grp * 32 + lane] = code;
  if (lane == 0) scales[drow * groups + grp] = (uint8_t)(exponent + 127);
}

// q [B, heads, D] bf16 (post-RoPE), ring codes [R, window, D] / scales [R, window, D/32], ring_ids [B],
// positions [B] (position of the query token; its K row is already in the ring), sink [heads] f32,
// inv_rotary [B, rope_tail] f32 = (cos, sin) of the inverse angle per adjacent pair, out [B, heads, D].
// grid (ceil(heads/16), B), 128 threads.
// SRC 0: keys from the FP8 ring as described above.
// SRC 1: keys are BF16 latent rows `rows_bf16` [num_rows, D] gathered through `indices` [B, width]
//        (entries < 0 are skipped): the sparse attention of a top-k selection (DSA); `window` = width,
//        `rings` = num_rows.
template <int SRC>
__global__ void __launch_bounds__(128)
latent_window_attention_kernel(const __nv_bfloat16* __restrict__ q, const uint8_t* __restrict__ codes,
                               const uint8_t* __restrict__ scales, const int* __restrict__ ring_ids,
                               const int* __restrict__ positions, const float* __restrict__ sink,
                               const float* __restrict__ inv_rotary, __nv_bfloat16* __restrict__ out, int heads, int D,
                               int window, int visible, int rings, int rope_tail, float scale, int round_p, int* status,
                               const __nv_bfloat16* __restrict__ rows_bf16, const int* __restrict__ indices) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t lw_smem[];
  const int chunks = D / 8;                       // 16-byte chunks per row
  uint8_t* sQ = lw_smem;                          // [16][D] bf16
  uint8_t* sK = sQ + 16 * D * 2;                  // [64][D] bf16
  float* sS = reinterpret_cast<float*>(sK + LW_KEYS * D * 2);        // [16][64]
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(sS + 16 * LW_KEYS);   // [16][64] (64 bf16 = 8 chunks per row)
  float* sM = reinterpret_cast<float*>(sP + 16 * LW_KEYS);           // running max [16]
  float* sL = sM + 16;                                               // running sum [16]
  float* sR = sL + 16;                                               // rescale of this block [16]
  const int b = blockIdx.y, h0 = blockIdx.x * 16;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  int nvis, first = 0;
  const uint8_t* rc = nullptr; const uint8_t* rs = nullptr;
  __shared__ int s_valid[LW_KEYS];
  if (SRC == 0) {
    const int ring = ring_ids[b], pos = positions[b];
    if (ring < 0 || ring >= rings || pos < 0) { if (tid == 0) set_status(status, KID_LATENT, FF_ERR_BOUNDS, b, ring); return; }
    // the last `visible` positions up to `pos`; a ring longer than that keeps the rows of later positions of the same
    // launch (prefill chunks) out of the way of the rows an earlier query still reads
    nvis = min(pos + 1, visible);
    first = (pos + 1 - nvis) % window;
    rc = codes + (size_t)ring * window * D;
    rs = scales + (size_t)ring * window * (D / 32);
  } else {
    nvis = window;
  }

  // Q tile (rows beyond `heads` are zero)
  for (int i = tid; i < 16 * chunks; i += 128) {
    const int r = i / chunks, c = i - r * chunks;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + r < heads) v = *reinterpret_cast<const uint4*>(q + ((size_t)b * heads + h0 + r) * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + lw_off(r, c, chunks)) = v;
  }
  if (tid < 16) { sM[tid] = -INFINITY; sL[tid] = 0.f; }
  const int ndw = D / 4;                          // output dims owned by a warp
  float o[16][4];                                 // up to 128 dims per warp: n-tile i covers dims warp*ndw + 8i .. +7
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const uint32_t sQa = smem_u32(sQ), sKa = smem_u32(sK), sPa = smem_u32(sP);
  __syncthreads();

  for (int k0 = 0; k0 < nvis; k0 += LW_KEYS) {
    const int nk = min(LW_KEYS, nvis - k0);
    if (SRC == 1) {
      // gather BF16 rows; an index < 0 (or out of range, flagged) leaves a zero row and a masked score
      if (tid < LW_KEYS) {
        int idx = (tid < nk) ? indices[(size_t)b * window + k0 + tid] : -1;
        if (idx >= rings) { set_status(status, KID_DSA, FF_ERR_BOUNDS, b, idx); idx = -1; }
        s_valid[tid] = idx;
      }
      __syncthreads();
      for (int i = tid; i < LW_KEYS * chunks; i += 128) {
        const int key = i / chunks, c = i - key * chunks;
        const int idx = s_valid[key];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (idx >= 0) v = *reinterpret_cast<const uint4*>(rows_bf16 + (size_t)idx * D + c * 8);
        *reinterpret_cast<uint4*>(sK + lw_off(key, c, chunks)) = v;
      }
    } else
    // de-quantise the block: one 16-code vector per thread step
    for (int i = tid; i < LW_KEYS * (D / 16); i += 128) {
      const int key = i / (D / 16), v16 = i - key * (D / 16);
      uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
      if (key < nk) {
        const int slot = (first + k0 + key) % window;
        const uint4 cv = *reinterpret_cast<const uint4*>(rc + (size_t)slot * D + v16 * 16);
        const float sc = lw_e8m0(rs[(size_t)slot * (D / 32) + v16 / 2]);
        const uint8_t* cb = reinterpret_cast<const uint8_t*>(&cv);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(lw_e4m3(cb[2 * j]) * sc, lw_e4m3(cb[2 * j + 1]) * sc);
        lo = make_uint4(w[0], w[1], w[2], w[3]); hi = make_uint4(w[4], w[5], w[6], w[7]);
      }
      *reinterpret_cast<uint4*>(sK + lw_off(key, 2 * v16, chunks)) = lo;
      *reinterpret_cast<uint4*>(sK + lw_off(key, 2 * v16 + 1, chunks)) = hi;
    }
    __syncthreads();
    // S[16 heads][16 keys of this warp]
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4], b0, b1, b2, b3;
      lw_ldsm4(sQa + lw_off((lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4), chunks), a[0], a[1], a[2], a[3]);
      lw_ldsm4(sKa + lw_off(warp * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1), chunks), b0, b1, b2, b3);
      lw_mma(s[0], a, b0, b1);
      lw_mma(s[1], a, b2, b3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = warp * 16 + i * 8 + 2 * t + (j & 1), row = g + ((j >> 1) << 3);
        const bool live = key < nk && (SRC == 0 || s_valid[key] >= 0);
        sS[row * LW_KEYS + key] = live ? s[i][j] * scale : -INFINITY;
      }
    __syncthreads();
    // soft-max bookkeeping: 8 threads per head row, 8 keys each
    {
      const int row = tid >> 3, part = tid & 7;
      float sc8[8], mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) { sc8[j] = sS[row * LW_KEYS + part * 8 + j]; mx = fmaxf(mx, sc8[j]); }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1)); mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float mprev = sM[row], bmax = fmaxf(mprev, mx);      // -inf only while every key so far was masked
      float bsum = 0.f;
      uint32_t pw[4];
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const float p0 = (sc8[j] == -INFINITY) ? 0.f : expf(sc8[j] - bmax);
        const float p1 = (sc8[j + 1] == -INFINITY) ? 0.f : expf(sc8[j + 1] - bmax);
        bsum += p0 + p1;
        pw[j >> 1] = pack_bf16x2(p0, p1);
      }
      bsum += __shfl_xor_sync(0xffffffffu, bsum, 1); bsum += __shfl_xor_sync(0xffffffffu, bsum, 2);
      bsum += __shfl_xor_sync(0xffffffffu, bsum, 4);
      // P tile [16][64] bf16: 8 chunks per row, chunk `part` XOR row
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(sP) + lw_off(row, part, 8)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      __syncwarp();
      if (part == 0) {
        const float resc = (k0 == 0 || mprev == -INFINITY) ? 1.f : expf(mprev - bmax);
        sR[row] = resc;
        sL[row] = sL[row] * resc + bsum;
        sM[row] = bmax;
      }
    }
    __syncthreads();
    // O[16][dims of this warp] = O * rescale + P V
    {
      const float r0 = sR[g], r1 = sR[g + 8];
      if (r0 != 1.f || r1 != 1.f) {
#pragma unroll
        for (int i = 0; i < 16; ++i) { o[i][0] *= r0; o[i][1] *= r0; o[i][2] *= r1; o[i][3] *= r1; }
      }
#pragma unroll
      for (int ks = 0; ks < LW_KEYS / 16; ++ks) {
        uint32_t pa[4];
        lw_ldsm4(sPa + lw_off((lane & 7) + (((lane >> 3) & 1) << 3), 2 * ks + (lane >> 4), 8), pa[0], pa[1], pa[2], pa[3]);
        const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          if (dp * 16 < ndw) {
            uint32_t b0, b1, b2, b3;
            lw_ldsm4t(sKa + lw_off(key, (warp * ndw) / 8 + dp * 2 + (lane >> 4), chunks), b0, b1, b2, b3);
            lw_mma(o[2 * dp], pa, b0, b1);
            lw_mma(o[2 * dp + 1], pa, b2, b3);
          }
        }
      }
    }
    __syncthreads();
  }
  // denominator with the sink, divide, BF16, inverse rotary on the tail, BF16
  const int tail = D - rope_tail;
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int row = g + 8 * e, head = h0 + row;
    if (head >= heads) continue;
    const float denom = sL[row] + ((sM[row] == -INFINITY) ? 1.f : expf(sink[head] - sM[row]));   // no key: only the sink
    __nv_bfloat16* orow = out + ((size_t)b * heads + head) * D;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i * 8 >= ndw) continue;
      const int d = warp * ndw + i * 8 + 2 * t;
      float a = __bfloat162float(__float2bfloat16(o[i][2 * e] / denom));
      float c = __bfloat162float(__float2bfloat16(o[i][2 * e + 1] / denom));
      if (d >= tail) {
        const float* ir = inv_rotary + (size_t)b * rope_tail + (d - tail);
        const float cs = ir[0], sn = ir[1];
        const float a2 = a * cs - c * sn, c2 = a * sn + c * cs;
        a = a2; c = c2;
      }
      *reinterpret_cast<uint32_t*>(orow + d) = pack_bf16x2(a, c);
    }
  }
  (void)round_p;
}

// Rotary embedding on the tail of every head: x [rows, heads * D] bf16 (row stride ldx), the adjacent pairs
// (2p, 2p + 1) of the last `tail` dims of a head are rotated by the angle whose (cos, sin) is cs[row, 2p .. 2p + 1].
// The forward rotation of the queries and of the latent key row before the ring write (the reference's
// rope_pair_rows / rope_pair_tail, kernels/rope_kv.cu); the attention kernel above applies the inverse to its output.
__global__ void rope_pair_tail_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, long long rows, int heads,
                                      int D, int ldx, int tail) {
  pdl_trigger();
  pdl_wait();
  const int half = tail / 2;
  const long long total = rows * heads * half;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i % half);
    const long long rh = i / half;
    const int h = (int)(rh % heads);
    const long long row = rh / heads;
    __nv_bfloat162* ptr = reinterpret_cast<__nv_bfloat162*>(x + row * ldx + (size_t)h * D + (D - tail) + 2 * p);
    const float2 c = *reinterpret_cast<const float2*>(cs + row * tail + 2 * p);
    const float2 v = __bfloat1622float2(*ptr);
    *ptr = __floats2bfloat162_rn(v.x * c.x - v.y * c.y, v.x * c.y + v.y * c.x);
  }
}

}  // namespace ff
using namespace ff;

// Quantise rows per 32 to E4M3 + E8M0. ring_ids/positions null: linear codes [rows, D] / scales [rows, D/32];
// otherwise row r is written to slot positions[r] % window of ring ring_ids[r] (codes [rings, window, D]).
FF_EXPORT int ff_latent_quant(const void* x, void* codes, void* scales, const int* ring_ids, const int* positions,
                              long long rows, int D, int ldx, int window, int rings, int* status, cudaStream_t s) {
  if (rows <= 0 || D <= 0 || D % 32 || ldx < D) return FF_HOST_BAD_SHAPE;
  if ((ring_ids == nullptr) != (positions == nullptr)) return FF_HOST_BAD_SHAPE;
  if (ring_ids != nullptr && (window <= 0 || rings <= 0)) return FF_HOST_BAD_SHAPE;
  const long long warps = rows * (D / 32);
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (int lr = launch_pdl(latent_quant_kernel, dim3(blocks), dim3(256), 0, s, 0, (const __nv_bfloat16*)x, (uint8_t*)codes,
                          (uint8_t*)scales, ring_ids, positions, rows, D, ldx, window, rings, status)) return lr;
  return launch_result();
}

FF_EXPORT int ff_latent_window_attention(const void* q, const void* codes, const void* scales, const int* ring_ids,
                                         const int* positions, const float* sink, const float* inv_rotary, void* out,
                                         int batch, int heads, int D, int window, int visible, int rings, int rope_tail,
                                         float scale, int* status, cudaStream_t s) {
  if (batch <= 0 || heads <= 0 || D <= 0 || D % 64 || D > LW_MAXD || window <= 0 || rings <= 0) return FF_HOST_BAD_SHAPE;
  if (visible <= 0 || visible > window) return FF_HOST_BAD_SHAPE;
  if (rope_tail < 0 || rope_tail > D || rope_tail % 2 || !(scale > 0.f)) return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(codes) & 15)) return FF_HOST_BAD_ALIGN;
  const int smem = 16 * D * 2 + LW_KEYS * D * 2 + 16 * LW_KEYS * 4 + 16 * LW_KEYS * 2 + 3 * 16 * 4;
  if (int r = opt_in_smem(latent_window_attention_kernel<0>, smem)) return r;
  dim3 grid((heads + 15) / 16, batch);
  if (int lr = launch_pdl(latent_window_attention_kernel<0>, grid, dim3(128), smem, s, 0, (const __nv_bfloat16*)q,
                          (const uint8_t*)codes, (const uint8_t*)scales, ring_ids, positions, sink, inv_rotary,
                          (__nv_bfloat16*)out, heads, D, window, visible, rings, rope_tail, scale, 1, status, nullptr,
                          nullptr)) return lr;
  return launch_result();
}

// Sparse attention over a selection: out[r, h] = softmax_with_sink(q[r, h] . latent[idx]) latent[idx] for
// idx in indices[r, :] (entries < 0 skipped). q / out [rows, heads, D] bf16, latent [num_rows, D] bf16,
// indices [rows, width] int32, sink [heads] f32. The direct latent form of the reference's
// dsa_sparse_attention_direct (kernels/dsa.cu:366-425), all heads of a row sharing one gathered tile.
FF_EXPORT int ff_latent_sparse_attention(const void* q, const void* latent, const int* indices, const float* sink, void* out,
                                         int rows, int heads, int D, int width, int num_rows, float scale, int* status,
                                         cudaStream_t s) {
  if (rows <= 0 || heads <= 0 || D <= 0 || D % 64 || D > LW_MAXD || width <= 0 || num_rows <= 0) return FF_HOST_BAD_SHAPE;
  if (!(scale > 0.f)) return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(latent) & 15)) return FF_HOST_BAD_ALIGN;
  const int smem = 16 * D * 2 + LW_KEYS * D * 2 + 16 * LW_KEYS * 4 + 16 * LW_KEYS * 2 + 3 * 16 * 4;
  if (int r = opt_in_smem(latent_window_attention_kernel<1>, smem)) return r;
  dim3 grid((heads + 15) / 16, rows);
  if (int lr = launch_pdl(latent_window_attention_kernel<1>, grid, dim3(128), smem, s, 0, (const __nv_bfloat16*)q,
                          (const uint8_t*)nullptr, (const uint8_t*)nullptr, (const int*)nullptr, (const int*)nullptr, sink,
                          (const float*)nullptr, (__nv_bfloat16*)out, heads, D, width, width, num_rows, 0, scale, 1, status,
                          (const __nv_bfloat16*)latent, indices)) return lr;
  return launch_result();
}

// In-place rotary on the last `tail` dims of every head (adjacent pairs); cs [rows, tail] f32 = (cos, sin) per pair.
FF_EXPORT int ff_rope_pair_tail(void* x, const float* cs, long long rows, int heads, int D, int ldx, int tail,
                                cudaStream_t s) {
  if (rows <= 0 || heads <= 0 || D <= 0 || tail <= 0 || tail > D || (tail & 1) || (D & 1) || (ldx & 1) || ldx < heads * D)
    return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) & 3) || (reinterpret_cast<uintptr_t>(cs) & 7)) return FF_HOST_BAD_ALIGN;
  const long long total = rows * heads * (tail / 2);
  const unsigned blocks = (unsigned)std::min<long long>((total + 255) / 256, 148 * 8);
  if (int lr = launch_pdl(rope_pair_tail_kernel, dim3(blocks), dim3(256), 0, s, 0, (__nv_bfloat16*)x, cs, rows, heads, D,
                          ldx, tail)) return lr;
  return launch_result();
}
