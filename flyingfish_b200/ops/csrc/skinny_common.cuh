// Pieces shared by the decode-shape GEMM kernels (gemm_skinny.cu, gemm_chain.cu): tile geometry,
// the stream-K unit -> (tile, k-block) walk, and the row-wise epilogues (SwiGLU; rotary embedding
// + paged KV-cache write) applied to a finished 128-row weight tile.
#pragma once
#include "ptx.cuh"

namespace ff {

constexpr int STOK = 128;         // token lanes of the accumulator (UMMA M)
constexpr int SBN = 256;          // most weight rows per tile (UMMA N)
constexpr int SBK = 64;           // k-block: 64 bf16 = one 128-byte swizzle row

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

// Row-wise epilogues over a 128-row weight tile whose first 64 columns pair with its last 64:
//   mode 1  SwiGLU: columns [0,64) are gate, [64,128) the matching up values (weight interleaved per
//           64 rows); output column tile*64 + j = silu(gate_j) * up_j, N/2 output columns.
//   mode 2  rotary embedding + KV-cache write for a fused QKV projection with 128-dim heads: the tile
//           is one head; Q and K heads are rotated (pairs j, j + 64), Q/K/V go to Y and K/V also to
//           their slot of the paged cache.
// Both round the accumulators to BF16 first and then do exactly what the stand-alone kernels
// (silu_mul, rope_kv_paged) do, so fused and unfused paths give the same bits.
struct SkinnyEpi {
  int mode;
  const float2* cos_sin;       // [rows, rot_dim/2] (cos, sin) of position * inv_freq, rounded to BF16 (ff_rope_table)
  const int* slots;
  __nv_bfloat16* kcache; __nv_bfloat16* vcache;
  int hq, hkv, rot_dim, block_size, num_blocks;
};

__device__ __forceinline__ float bf16r_sk(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ float silu_sk(float x) { return x / (1.0f + __expf(-x)); }

// lo/hi: eight values each of token row t, tile columns [j8*8, j8*8+8) and [64 + j8*8, ...)
__device__ __forceinline__ void emit_pair(const SkinnyEpi& ep, __nv_bfloat16* __restrict__ Y, int N, int ldy, int t, int tile,
                                          int j8, const float* lo, const float* hi, int* status) {
  if (ep.mode == 1) {
    const int col = tile * 64 + j8 * 8;
    if (col >= N / 2) return;
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a0 = bf16r_sk(silu_sk(bf16r_sk(lo[2 * j]))), a1 = bf16r_sk(silu_sk(bf16r_sk(lo[2 * j + 1])));
      o[j] = pack_bf16x2(a0 * bf16r_sk(hi[2 * j]), a1 * bf16r_sk(hi[2 * j + 1]));
    }
    *reinterpret_cast<uint4*>(Y + (size_t)t * ldy + col) = make_uint4(o[0], o[1], o[2], o[3]);
    return;
  }
  // mode 2
  const int head = tile;
  if (head >= ep.hq + 2 * ep.hkv) return;
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { a[j] = bf16r_sk(lo[j]); b[j] = bf16r_sk(hi[j]); }
  const bool is_v = head >= ep.hq + ep.hkv;
  if (!is_v) {
    const int rhalf = ep.rot_dim >> 1;
    const float2* tab = ep.cos_sin + (size_t)t * rhalf;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = j8 * 8 + j;
      if (i < rhalf) {
        const float2 c_s = tab[i];
        const float cs = c_s.x, sn = c_s.y;
        const float x1 = a[j], x2 = b[j];
        a[j] = bf16r_sk(bf16r_sk(x1 * cs) - bf16r_sk(x2 * sn));
        b[j] = bf16r_sk(bf16r_sk(x2 * cs) + bf16r_sk(x1 * sn));
      }
    }
  }
  const uint4 vlo = make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
  const uint4 vhi = make_uint4(pack_bf16x2(b[0], b[1]), pack_bf16x2(b[2], b[3]), pack_bf16x2(b[4], b[5]), pack_bf16x2(b[6], b[7]));
  __nv_bfloat16* y = Y + (size_t)t * ldy + (size_t)head * 128 + j8 * 8;
  *reinterpret_cast<uint4*>(y) = vlo;
  *reinterpret_cast<uint4*>(y + 64) = vhi;
  if (head >= ep.hq) {
    const int slot = ep.slots[t];
    if (slot < 0) return;                               // padding row: nothing cached
    const int blk = slot / ep.block_size, off = slot - blk * ep.block_size;
    if (blk >= ep.num_blocks) { set_status(status, KID_ROPE_KV, FF_ERR_BOUNDS, t, slot); return; }
    const int kvh = is_v ? head - ep.hq - ep.hkv : head - ep.hq;
    __nv_bfloat16* dst = (is_v ? ep.vcache : ep.kcache) + (((size_t)blk * ep.hkv + kvh) * ep.block_size + off) * 128 + j8 * 8;
    *reinterpret_cast<uint4*>(dst) = vlo;
    *reinterpret_cast<uint4*>(dst + 64) = vhi;
  }
}

}  // namespace ff
