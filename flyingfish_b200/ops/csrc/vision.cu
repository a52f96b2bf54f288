// Vision-tower and 3-D compute operators (no graphics API anywhere):
//   layernorm        : y = (x - mean) * rsqrt(var + eps) * w + b, FP32 statistics, one BF16 rounding
//   bias_act         : y = act(x + bias) in place; act 0 none, 1 tanh-GELU, 2 quick-GELU (x * sigmoid(1.702 x)),
//                      3 erf-GELU, 4 SiLU. The sum is rounded to BF16 before the activation (the projection's
//                      output dtype), the result once more.
//   voxel hash       : open-addressing table over (batch, x, y, z) keys built with atomicCAS (bounded probing),
//                      value = lowest row index holding the key (deterministic under duplicates)
//   neighbor_map     : for every site and every kernel offset, the row index of the neighbouring site or -1
//   sparse_gather    : rows gathered through a neighbour map into the im2col operand of a sparse convolution
//                      [sites, offsets * channels] (missing neighbours are zero rows); the convolution itself is one
//                      tensor-core GEMM with FP32 accumulation over offsets * channels
//   voxelize         : points -> integer voxel coordinates inside a grid (or -1 outside)
//   rotate_quant     : block-diagonal regular Hadamard rotation (kron of H4 / 2) of every `group` activations,
//                      per-row absmax INT8 quantisation: s = max(|xR|, 1e-12) / 127, q = rint(xR / s)
//   int8_linear      : y = bf16(dot_i32(q_x, q_w) * s_x[row] * s_w[col]) with dp4a
// The reference's counterparts are kernels/vision_ops.cu (sparse_gather*, vision_bias_gelu_f32,
// vision_bias_quick_gelu_f32), src/sparse.rs (site tables) and src/convrot.rs:1-60 (rotation and quantiser).
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

// ------------------------------------------------------------------------------------------------
// layernorm: one CTA (128 threads) per row, row cached in registers (<= 8 vectors of 8 per thread)
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_128(float v, float* s_red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) s_red[warp] = v;
  __syncthreads();
  return s_red[0] + s_red[1] + s_red[2] + s_red[3];
}

constexpr int LN_MAX_VEC = 8;          // hidden <= 128 * 8 * 8 = 8192

__global__ void __launch_bounds__(128)
layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                 const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, int hidden, int ldx, int ldy,
                 float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_red[4];
  const int row = blockIdx.x, nvec = hidden >> 3;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint4 v[LN_MAX_VEC];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * 128;
    if (idx < nvec) {
      v[i] = src[idx];
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(p[j]); sum += f.x + f.y; }
    }
  }
  const float mean = block_sum_128(sum, s_red) / (float)hidden;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < LN_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * 128;
    if (idx < nvec) {
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(p[j]);
        sq += (f.x - mean) * (f.x - mean) + (f.y - mean) * (f.y - mean);
      }
    }
  }
  const float rstd = rsqrtf(block_sum_128(sq, s_red) / (float)hidden + eps);
  uint4* dst = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
#pragma unroll
  for (int i = 0; i < LN_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * 128;
    if (idx < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[idx];
      uint4 bv = make_uint4(0u, 0u, 0u, 0u);
      if (b) bv = reinterpret_cast<const uint4*>(b)[idx];
      const uint32_t* p = reinterpret_cast<const uint32_t*>(&v[i]);
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
      const uint32_t* bp = reinterpret_cast<const uint32_t*>(&bv);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(p[j]), ww = unpack_bf16x2(wp[j]), bb = unpack_bf16x2(bp[j]);
        o[j] = pack_bf16x2((f.x - mean) * rstd * ww.x + bb.x, (f.y - mean) * rstd * ww.y + bb.y);
      }
      dst[idx] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// bias + activation, in place, 8 elements per thread
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float bfr_v(float x) { return __bfloat162float(__float2bfloat16(x)); }

__device__ __forceinline__ float act_apply(float x, int act) {
  switch (act) {
    case 1: return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 2: return x / (1.f + __expf(-1.702f * x));
    case 3: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case 4: return x / (1.f + __expf(-x));
    case 5: return fmaxf(x, 0.f);
    default: return x;
  }
}

__global__ void __launch_bounds__(256)
bias_act_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ bias, long long rows, int n, int ldx,
                int act) {
  pdl_trigger();
  pdl_wait();
  const int nvec = n >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= rows * nvec) return;
  const long long row = gid / nvec;
  const int c = (int)(gid - row * nvec);
  uint4* p = reinterpret_cast<uint4*>(x + (size_t)row * ldx) + c;
  uint4 v = *p;
  uint4 bv = make_uint4(0u, 0u, 0u, 0u);
  if (bias) bv = reinterpret_cast<const uint4*>(bias)[c];
  uint32_t* vp = reinterpret_cast<uint32_t*>(&v);
  const uint32_t* bp = reinterpret_cast<const uint32_t*>(&bv);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_bf16x2(vp[j]), bb = unpack_bf16x2(bp[j]);
    vp[j] = pack_bf16x2(act_apply(bfr_v(f.x + bb.x), act), act_apply(bfr_v(f.y + bb.y), act));
  }
  *p = v;
}

// y[row, c] = bf16(a[row, c] * sigmoid(gate[row, c])): the output gate of gated attention layers (the gate is a column
// slice of the fused projection, hence its own leading dimension)
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ gate, __nv_bfloat16* __restrict__ y,
                    long long rows, int n, int lda, int ldg, int ldy) {
  pdl_trigger();
  pdl_wait();
  const int nvec = n >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= rows * nvec) return;
  const long long row = gid / nvec;
  const int c = (int)(gid - row * nvec);
  const uint4 av = *(reinterpret_cast<const uint4*>(a + (size_t)row * lda) + c);
  const uint4 gv = *(reinterpret_cast<const uint4*>(gate + (size_t)row * ldg) + c);
  uint4 o;
  const uint32_t* ap = reinterpret_cast<const uint32_t*>(&av);
  const uint32_t* gp = reinterpret_cast<const uint32_t*>(&gv);
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 x = unpack_bf16x2(ap[j]), g = unpack_bf16x2(gp[j]);
    op[j] = pack_bf16x2(x.x / (1.f + __expf(-g.x)), x.y / (1.f + __expf(-g.y)));
  }
  *(reinterpret_cast<uint4*>(y + (size_t)row * ldy) + c) = o;
}

// ------------------------------------------------------------------------------------------------
// group norm over channels-last activations [n, positions, C] and dense 3-D convolution as im2col + GEMM
// (kernels/vision_ops.cu group-norm / im2col families of the reference, there channels-first)
// ------------------------------------------------------------------------------------------------
constexpr int GN_CHUNKS = 64;

// partial sums of one (sample, group, chunk of positions): part[((n * G + g) * GN_CHUNKS + chunk) * 2 + {0, 1}]
__global__ void __launch_bounds__(256)
group_norm_stats_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ part, int positions, int C, int G) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_a[8], s_b[8];
  const int chunk = blockIdx.x, g = blockIdx.y, n = blockIdx.z;
  const int cg = C / G;
  const int per = (positions + GN_CHUNKS - 1) / GN_CHUNKS;
  const int p0 = chunk * per, p1 = min(positions, p0 + per);
  const __nv_bfloat16* base = x + ((size_t)n * positions) * C + (size_t)g * cg;
  float sum = 0.f, sq = 0.f;
  const long long total = (long long)max(p1 - p0, 0) * cg;
  for (long long i = threadIdx.x; i < total; i += 256) {
    const int p = p0 + (int)(i / cg), c = (int)(i % cg);
    const float v = __bfloat162float(base[(size_t)p * C + c]);
    sum += v; sq = fmaf(v, v, sq);
  }
  sum = warp_sum(sum); sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) { s_a[threadIdx.x >> 5] = sum; s_b[threadIdx.x >> 5] = sq; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < 8; ++w) { a += s_a[w]; b += s_b[w]; }
    float* dst = part + (((size_t)n * G + g) * GN_CHUNKS + chunk) * 2;
    dst[0] = a; dst[1] = b;
  }
}

// y = act((x - mean) * rstd * w + b); the chunk partials are summed in chunk order by every thread that needs them
__global__ void __launch_bounds__(256)
group_norm_apply_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ part, const float* __restrict__ w,
                        const float* __restrict__ b, __nv_bfloat16* __restrict__ y, int positions, int C, int G, float eps,
                        int act, long long total8) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  if (gid >= total8) return;
  const int cv = C >> 3;
  const int c0 = (int)(gid % cv) * 8;
  const long long row = gid / cv;
  const int n = (int)(row / positions);
  const int cg = C / G;
  uint4 v = *reinterpret_cast<const uint4*>(x + (size_t)row * C + c0);
  uint32_t* vp = reinterpret_cast<uint32_t*>(&v);
  float mean = 0.f, rstd = 0.f;
  int cur = -1;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 f = unpack_bf16x2(vp[j]);
    float o[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = c0 + 2 * j + h;
      const int g = c / cg;
      if (g != cur) {
        const float* src = part + ((size_t)n * G + g) * GN_CHUNKS * 2;
        float a = 0.f, q = 0.f;
        for (int k = 0; k < GN_CHUNKS; ++k) { a += src[2 * k]; q += src[2 * k + 1]; }
        const float cnt = (float)positions * (float)cg;
        mean = a / cnt;
        rstd = rsqrtf(fmaxf(q / cnt - mean * mean, 0.f) + eps);
        cur = g;
      }
      const float xv = h == 0 ? f.x : f.y;
      o[h] = act_apply(fmaf((xv - mean) * rstd, w[c], b ? b[c] : 0.f), act);
    }
    vp[j] = pack_bf16x2(o[0], o[1]);
  }
  *reinterpret_cast<uint4*>(y + (size_t)row * C + c0) = v;
}

// cols[((n, d, h, w), tap, c)] = x[n, d + kd - pad, h + kh - pad, w + kw - pad, c] (zero outside), taps in (kd, kh, kw)
// order; one thread per (output position, tap, 8 channels)
__global__ void __launch_bounds__(256)
im2col3d_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ cols, int D, int H, int W, int C, int k,
                int pad, long long total8) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  if (gid >= total8) return;
  const int cv = C >> 3, taps = k * k * k;
  const int c0 = (int)(gid % cv) * 8;
  long long r = gid / cv;
  const int tap = (int)(r % taps); r /= taps;
  const int w = (int)(r % W); r /= W;
  const int h = (int)(r % H); r /= H;
  const int d = (int)(r % D);
  const long long n = r / D;
  const int kd = tap / (k * k), kh = (tap / k) % k, kw = tap % k;
  const int sd = d + kd - pad, sh = h + kh - pad, sw = w + kw - pad;
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (sd >= 0 && sd < D && sh >= 0 && sh < H && sw >= 0 && sw < W)
    v = *reinterpret_cast<const uint4*>(x + ((((size_t)n * D + sd) * H + sh) * W + sw) * C + c0);
  *reinterpret_cast<uint4*>(cols + (size_t)gid * 8) = v;
}

// Neighbourhood attention over a 2-D grid: the query at (i, j) attends to the ks x ks keys of the window centred on it,
// shifted inwards at the borders so that it always holds ks x ks positions. q, k, v, out: [n, H, W, heads, d] BF16.
// One warp per (query, head): lanes split the head dimension (d <= 256, d % 32 == 0), online soft-max over the window.
__global__ void __launch_bounds__(256)
neighborhood_attn_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                         const __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ out, int H, int W, int heads, int d,
                         int ks, float scale_log2, long long total) {
  pdl_trigger();
  pdl_wait();
  const long long wid = ((long long)blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= total) return;
  const int hd = (int)(wid % heads);
  long long r = wid / heads;
  const int j = (int)(r % W); r /= W;
  const int i = (int)(r % H);
  const long long n = r / H;
  const int per = d >> 5;                              // dims per lane (1..8)
  const int i0 = min(max(i - ks / 2, 0), H - ks), j0 = min(max(j - ks / 2, 0), W - ks);
  const size_t stride = (size_t)heads * d;
  const __nv_bfloat16* qp = q + (((size_t)n * H + i) * W + j) * stride + (size_t)hd * d + lane * per;
  float qv[8], acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) { qv[e] = e < per ? __bfloat162float(qp[e]) : 0.f; acc[e] = 0.f; }
  float m = -INFINITY, l = 0.f;
  for (int a = 0; a < ks; ++a)
    for (int b = 0; b < ks; ++b) {
      const size_t off = (((size_t)n * H + i0 + a) * W + j0 + b) * stride + (size_t)hd * d + lane * per;
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) if (e < per) dot = fmaf(qv[e], __bfloat162float(k[off + e]), dot);
      dot = warp_sum(dot) * scale_log2;
      const float mn = fmaxf(m, dot);
      const float corr = exp2f(m - mn), p = exp2f(dot - mn);
      l = l * corr + p;
#pragma unroll
      for (int e = 0; e < 8; ++e) if (e < per) acc[e] = fmaf(p, __bfloat162float(v[off + e]), acc[e] * corr);
      m = mn;
    }
  const float inv = 1.f / l;
  __nv_bfloat16* op = out + (((size_t)n * H + i) * W + j) * stride + (size_t)hd * d + lane * per;
#pragma unroll
  for (int e = 0; e < 8; ++e) if (e < per) op[e] = __float2bfloat16(acc[e] * inv);
}

// ------------------------------------------------------------------------------------------------
// voxel hash table. key = (b:16 | x:16 | y:16 | z:16) of non-negative coordinates < 65536; slot value =
// lowest row index with that key. Empty key = all ones.
// ------------------------------------------------------------------------------------------------
constexpr unsigned long long HASH_EMPTY = ~0ull;

__device__ __forceinline__ unsigned long long voxel_key(int4 c) {
  return ((unsigned long long)(c.x & 0xffff) << 48) | ((unsigned long long)(c.y & 0xffff) << 32) |
         ((unsigned long long)(c.z & 0xffff) << 16) | (unsigned long long)(c.w & 0xffff);
}
__device__ __forceinline__ unsigned int hash64(unsigned long long k) {
  k ^= k >> 33; k *= 0xff51afd7ed558ccdull; k ^= k >> 33; k *= 0xc4ceb9fe1a85ec53ull; k ^= k >> 33;
  return (unsigned int)k;
}
__device__ __forceinline__ bool coord_ok(int4 c) {
  return c.x >= 0 && c.y >= 0 && c.z >= 0 && c.w >= 0 && c.x < 65536 && c.y < 65536 && c.z < 65536 && c.w < 65536;
}

__global__ void hash_build_kernel(const int4* __restrict__ coords, int n, unsigned long long* __restrict__ keys,
                                  int* __restrict__ vals, unsigned int cap_mask, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 c = coords[i];
  if (!coord_ok(c)) return;                                   // rows outside the key range are never found
  const unsigned long long k = voxel_key(c);
  unsigned int h = hash64(k) & cap_mask;
  for (unsigned int probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long prev = atomicCAS(&keys[h], HASH_EMPTY, k);
    if (prev == HASH_EMPTY || prev == k) { atomicMin(&vals[h], i); return; }
    h = (h + 1) & cap_mask;
  }
  set_status(status, KID_VISION, FF_ERR_CAPACITY, i, (int)cap_mask);
}

__device__ __forceinline__ int hash_find(const unsigned long long* __restrict__ keys, const int* __restrict__ vals,
                                         unsigned int cap_mask, int4 c) {
  if (!coord_ok(c)) return -1;
  const unsigned long long k = voxel_key(c);
  unsigned int h = hash64(k) & cap_mask;
  for (unsigned int probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long cur = keys[h];
    if (cur == k) return vals[h];
    if (cur == HASH_EMPTY) return -1;
    h = (h + 1) & cap_mask;
  }
  return -1;
}

// nbr [n_off, n]: row of the site at coords[i] + offsets[o] (same batch), or -1
__global__ void neighbor_map_kernel(const int4* __restrict__ coords, int n, const int4* __restrict__ offsets, int n_off,
                                    const unsigned long long* __restrict__ keys, const int* __restrict__ vals,
                                    unsigned int cap_mask, int* __restrict__ nbr) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)n * n_off) return;
  const int o = (int)(gid / n), i = (int)(gid - (long long)o * n);
  const int4 c = coords[i], d = offsets[o];
  nbr[gid] = hash_find(keys, vals, cap_mask, make_int4(c.x, c.y + d.y, c.z + d.z, c.w + d.w));
}

// first[i] = 1 when row i is the lowest row with its key (unique-site selection)
__global__ void hash_first_kernel(const int4* __restrict__ coords, int n, const unsigned long long* __restrict__ keys,
                                  const int* __restrict__ vals, unsigned int cap_mask, int* __restrict__ first) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  first[i] = hash_find(keys, vals, cap_mask, coords[i]) == i ? 1 : 0;
}

// out [n, n_off * C]: block o of row i = feat[nbr[o, i]] or zeros. One thread per 16-byte vector.
__global__ void __launch_bounds__(256)
sparse_gather_kernel(const __nv_bfloat16* __restrict__ feat, const int* __restrict__ nbr, int n, int n_off, int C,
                     int n_src, __nv_bfloat16* __restrict__ out, int* status) {
  const int cvec = C >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)n * n_off * cvec;
  if (gid >= total) return;
  const int v = (int)(gid % cvec);
  const int o = (int)((gid / cvec) % n_off);
  const int i = (int)(gid / ((long long)cvec * n_off));
  const int src = nbr[(size_t)o * n + i];
  uint4 val = make_uint4(0u, 0u, 0u, 0u);
  if (src >= n_src) set_status(status, KID_VISION, FF_ERR_BOUNDS, i, src);
  else if (src >= 0) val = __ldg(reinterpret_cast<const uint4*>(feat + (size_t)src * C) + v);
  reinterpret_cast<uint4*>(out + ((size_t)i * n_off + o) * C)[v] = val;
}

// coords[i] = (batch[i], floor((p - origin) / voxel)) when inside [0, dims), else (-1, -1, -1, -1)
__global__ void voxelize_kernel(const float* __restrict__ pts, const int* __restrict__ batch, int n, float ox, float oy,
                                float oz, float inv_voxel, int dx, int dy, int dz, int4* __restrict__ coords) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int x = (int)floorf((pts[3 * i] - ox) * inv_voxel);
  const int y = (int)floorf((pts[3 * i + 1] - oy) * inv_voxel);
  const int z = (int)floorf((pts[3 * i + 2] - oz) * inv_voxel);
  const bool in = x >= 0 && y >= 0 && z >= 0 && x < dx && y < dy && z < dz;
  coords[i] = in ? make_int4(batch ? batch[i] : 0, x, y, z) : make_int4(-1, -1, -1, -1);
}

// ------------------------------------------------------------------------------------------------
// Hadamard rotate + INT8 quantise: one CTA (128 threads) per row, the row in shared memory as FP32.
// Stage with stride s: every quadruple (i, i+s, i+2s, i+3s) inside a block of 4s -> H4 / 2 times it.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
rotate_quant_kernel(const __nv_bfloat16* __restrict__ x, int k, int group, int ldx, int8_t* __restrict__ codes,
                    float* __restrict__ scales) {
  extern __shared__ float rq_s[];
  __shared__ float s_red[4];
  const int row = blockIdx.x;
  for (int i = threadIdx.x; i < k; i += 128) rq_s[i] = __bfloat162float(x[(size_t)row * ldx + i]);
  __syncthreads();
  for (int s = group >> 2; s >= 1; s >>= 2) {
    for (int q = threadIdx.x; q < (k >> 2); q += 128) {
      const int blk = q / s, in = q - blk * s;
      const int i0 = blk * 4 * s + in;
      const float a = rq_s[i0], b = rq_s[i0 + s], c = rq_s[i0 + 2 * s], d = rq_s[i0 + 3 * s];
      // column j of H4 = [[1,1,1,-1],[1,1,-1,1],[1,-1,1,1],[-1,1,1,1]] applied to the row vector (a b c d)
      rq_s[i0] = 0.5f * (a + b + c - d);
      rq_s[i0 + s] = 0.5f * (a + b - c + d);
      rq_s[i0 + 2 * s] = 0.5f * (a - b + c + d);
      rq_s[i0 + 3 * s] = 0.5f * (-a + b + c + d);
    }
    __syncthreads();
  }
  float amax = 0.f;
  for (int i = threadIdx.x; i < k; i += 128) {
    const float r = bfr_v(rq_s[i]);                            // the rotated activation is a BF16 value
    rq_s[i] = r;
    amax = fmaxf(amax, fabsf(r));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  const float sc = fmaxf(amax, 1e-12f) / 127.f;
  if (threadIdx.x == 0) scales[row] = sc;
  for (int i = threadIdx.x; i < k; i += 128) {
    const float q = rintf(rq_s[i] / sc);
    codes[(size_t)row * k + i] = (int8_t)fminf(fmaxf(q, -127.f), 127.f);
  }
}

// y[row, col] = bf16(dot_i32 * sx[row] * sw[col]); one warp per (row, 4 columns), lanes split k in 16-byte vectors
__global__ void __launch_bounds__(256)
int8_linear_kernel(const int8_t* __restrict__ qx, const float* __restrict__ sx, const int8_t* __restrict__ qw,
                   const float* __restrict__ sw, __nv_bfloat16* __restrict__ y, int rows, int n, int k, int ldy) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int col_groups = (n + 3) >> 2;
  if (warp >= rows * col_groups) return;
  const int row = warp / col_groups, c0 = (warp - row * col_groups) * 4;
  const int4* xv = reinterpret_cast<const int4*>(qx + (size_t)row * k);
  int acc[4] = {0, 0, 0, 0};
  for (int v = lane; v < (k >> 4); v += 32) {
    const int4 a = xv[v];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (c0 + j < n) {
        const int4 b = __ldg(reinterpret_cast<const int4*>(qw + (size_t)(c0 + j) * k) + v);
        acc[j] = __dp4a(a.x, b.x, acc[j]); acc[j] = __dp4a(a.y, b.y, acc[j]);
        acc[j] = __dp4a(a.z, b.z, acc[j]); acc[j] = __dp4a(a.w, b.w, acc[j]);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
  }
  if (lane < 4 && c0 + lane < n)
    y[(size_t)row * ldy + c0 + lane] = __float2bfloat16((float)acc[lane] * sx[row] * sw[c0 + lane]);
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_layernorm(const void* x, const void* w, const void* b, void* y, int rows, int hidden, int ldx, int ldy,
                           float eps, cudaStream_t s) {
  if (rows <= 0 || hidden <= 0 || hidden % 8 || hidden > 128 * 8 * LN_MAX_VEC || ldx % 8 || ldy % 8) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(layernorm_kernel, dim3(rows), dim3(128), 0, s, 0, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                          (const __nv_bfloat16*)b, (__nv_bfloat16*)y, hidden, ldx, ldy, eps)) return lr;
  return launch_result();
}

FF_EXPORT int ff_bias_act(void* x, const void* bias, long long rows, int n, int ldx, int act, cudaStream_t s) {
  if (rows <= 0 || n <= 0 || n % 8 || ldx % 8 || act < 0 || act > 5) return FF_HOST_BAD_SHAPE;
  const long long total = rows * (n / 8);
  if (int lr = launch_pdl(bias_act_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, (__nv_bfloat16*)x,
                          (const __nv_bfloat16*)bias, rows, n, ldx, act)) return lr;
  return launch_result();
}

FF_EXPORT int ff_sigmoid_gate(const void* a, const void* gate, void* y, long long rows, int n, int lda, int ldg, int ldy,
                              cudaStream_t s) {
  if (rows <= 0 || n <= 0 || n % 8 || lda % 8 || ldg % 8 || ldy % 8) return FF_HOST_BAD_SHAPE;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(gate) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return FF_HOST_BAD_ALIGN;
  const long long total = rows * (n / 8);
  if (int lr = launch_pdl(sigmoid_gate_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)a, (const __nv_bfloat16*)gate, (__nv_bfloat16*)y, rows, n, lda, ldg, ldy))
    return lr;
  return launch_result();
}

// x, y: [n, positions, C] BF16; w, b: [C] FP32; part: FP32 scratch of n * G * 64 * 2 floats. act as in ff_bias_act.
FF_EXPORT int ff_group_norm(const void* x, const float* w, const float* b, void* y, float* part, int n, int positions, int C,
                            int G, float eps, int act, cudaStream_t s) {
  if (n <= 0 || positions <= 0 || C <= 0 || G <= 0 || C % G || C % 8 || act < 0 || act > 5) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(group_norm_stats_kernel, dim3(GN_CHUNKS, G, n), dim3(256), 0, s, 0, (const __nv_bfloat16*)x, part,
                          positions, C, G)) return lr;
  const long long total8 = (long long)n * positions * (C / 8);
  if (int lr = launch_pdl(group_norm_apply_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)x, (const float*)part, w, b, (__nv_bfloat16*)y, positions, C, G, eps, act,
                          total8)) return lr;
  return launch_result();
}

FF_EXPORT int ff_neighborhood_attn(const void* q, const void* k, const void* v, void* out, int n, int H, int W, int heads,
                                   int d, int ks, float scale, cudaStream_t s) {
  if (n <= 0 || H <= 0 || W <= 0 || heads <= 0 || d <= 0 || d % 32 || d > 256 || ks < 1 || ks % 2 == 0 || ks > H || ks > W || !(scale > 0.f))
    return FF_HOST_BAD_SHAPE;
  const long long total = (long long)n * H * W * heads;
  if (int lr = launch_pdl(neighborhood_attn_kernel, dim3((unsigned)((total * 32 + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)out, H, W,
                          heads, d, ks, scale * 1.4426950408889634f, total)) return lr;
  return launch_result();
}

FF_EXPORT int ff_im2col3d(const void* x, void* cols, int n, int D, int H, int W, int C, int k, int pad, cudaStream_t s) {
  if (n <= 0 || D <= 0 || H <= 0 || W <= 0 || C <= 0 || C % 8 || k < 1 || k > 7 || pad < 0) return FF_HOST_BAD_SHAPE;
  const long long total8 = (long long)n * D * H * W * k * k * k * (C / 8);
  if (int lr = launch_pdl(im2col3d_kernel, dim3((unsigned)((total8 + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)x, (__nv_bfloat16*)cols, D, H, W, C, k, pad, total8)) return lr;
  return launch_result();
}

// keys: uint64[capacity], vals: int32[capacity]; capacity a power of two >= 2 * n. Both are initialised here.
FF_EXPORT int ff_voxel_hash_build(const int* coords, int n, unsigned long long* keys, int* vals, int capacity,
                                  int* status, cudaStream_t s) {
  if (n <= 0 || capacity < 2 * n || (capacity & (capacity - 1))) return FF_HOST_BAD_SHAPE;
  cudaError_t e = cudaMemsetAsync(keys, 0xff, (size_t)capacity * 8, s);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(vals, 0x7f, (size_t)capacity * 4, s);
  if (e != cudaSuccess) return (int)e;
  hash_build_kernel<<<(n + 255) / 256, 256, 0, s>>>(reinterpret_cast<const int4*>(coords), n, keys, vals,
                                                    (unsigned int)capacity - 1, status);
  return launch_result();
}

FF_EXPORT int ff_voxel_neighbor_map(const int* coords, int n, const int* offsets, int n_off, const unsigned long long* keys,
                                    const int* vals, int capacity, int* nbr, cudaStream_t s) {
  if (n <= 0 || n_off <= 0 || (capacity & (capacity - 1))) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)n * n_off;
  neighbor_map_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(reinterpret_cast<const int4*>(coords), n,
      reinterpret_cast<const int4*>(offsets), n_off, keys, vals, (unsigned int)capacity - 1, nbr);
  return launch_result();
}

FF_EXPORT int ff_voxel_first(const int* coords, int n, const unsigned long long* keys, const int* vals, int capacity,
                             int* first, cudaStream_t s) {
  if (n <= 0 || (capacity & (capacity - 1))) return FF_HOST_BAD_SHAPE;
  hash_first_kernel<<<(n + 255) / 256, 256, 0, s>>>(reinterpret_cast<const int4*>(coords), n, keys, vals,
                                                    (unsigned int)capacity - 1, first);
  return launch_result();
}

FF_EXPORT int ff_sparse_gather(const void* feat, const int* nbr, int n, int n_off, int C, int n_src, void* out, int* status,
                               cudaStream_t s) {
  if (n <= 0 || n_off <= 0 || C <= 0 || C % 8) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)n * n_off * (C / 8);
  sparse_gather_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>((const __nv_bfloat16*)feat, nbr, n, n_off, C, n_src,
                                                                       (__nv_bfloat16*)out, status);
  return launch_result();
}

FF_EXPORT int ff_voxelize(const float* pts, const int* batch, int n, float ox, float oy, float oz, float voxel, int dx,
                          int dy, int dz, int* coords, cudaStream_t s) {
  if (n <= 0 || !(voxel > 0.f) || dx <= 0 || dy <= 0 || dz <= 0 || dx > 65536 || dy > 65536 || dz > 65536)
    return FF_HOST_BAD_SHAPE;
  voxelize_kernel<<<(n + 255) / 256, 256, 0, s>>>(pts, batch, n, ox, oy, oz, 1.0f / voxel, dx, dy, dz,
                                                  reinterpret_cast<int4*>(coords));
  return launch_result();
}

FF_EXPORT int ff_rotate_quant(const void* x, int rows, int k, int group, int ldx, signed char* codes, float* scales,
                              cudaStream_t s) {
  bool pow4 = group >= 4 && !(group & (group - 1));
  if (pow4) { int t = 0; for (int g = group; g > 1; g >>= 1) ++t; pow4 = (t % 2) == 0; }
  if (rows <= 0 || k <= 0 || !pow4 || k % group || k * 4 > 200 * 1024) return FF_HOST_BAD_SHAPE;
  static int smem_set = 0;
  if (k * 4 > 48 * 1024 && smem_set < k * 4) {
    if (int r = opt_in_smem(rotate_quant_kernel, k * 4)) return r;
    smem_set = k * 4;
  }
  rotate_quant_kernel<<<rows, 128, (size_t)k * 4, s>>>((const __nv_bfloat16*)x, k, group, ldx, (int8_t*)codes, scales);
  return launch_result();
}

FF_EXPORT int ff_int8_linear(const signed char* qx, const float* sx, const signed char* qw, const float* sw, void* y,
                             int rows, int n, int k, int ldy, cudaStream_t s) {
  if (rows <= 0 || n <= 0 || k <= 0 || k % 16) return FF_HOST_BAD_SHAPE;
  const long long warps = (long long)rows * ((n + 3) / 4);
  int8_linear_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, s>>>((const int8_t*)qx, sx, (const int8_t*)qw, sw,
                                                                           (__nv_bfloat16*)y, rows, n, k, ldy);
  return launch_result();
}
