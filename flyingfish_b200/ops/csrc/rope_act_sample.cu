// Element-wise / row-wise operators of the decoder layer that are bound by memory traffic:
//   rope_kv_paged  : rotate-half RoPE on Q and K inside the packed QKV row, K/V written into the
//                    paged cache [block][kv_head][block_size][head_dim]
//   silu_mul       : SwiGLU activation with the reference's rounding modes
//   argmax_rows    : greedy sampling, ties -> lower id (optionally emits (value, id) pairs for a
//                    vocab-parallel merge)
//   sample_rows    : temperature / top-k / top-p / repetition penalty + Philox4x32-10 categorical
// Contracts follow kernels/rope_kv.cu:34-53, kernels/act.cu:220-262, kernels/sample.cu:3-6,276-279
// and src/sampling.rs:4-130 of the reference.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }

// One thread = one 16-byte vector pair (8 dims of the first half + the matching 8 dims of the
// second half) of one head of one row.
__global__ void rope_kv_paged_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slots, __nv_bfloat16* __restrict__ kcache,
                                     __nv_bfloat16* __restrict__ vcache, const float* __restrict__ inv_freq_tab,
                                     int rows, int hq, int hkv, int dim, int rot_dim, int block_size, int num_blocks,
                                     float theta, int ldqkv, int* status, const float2* __restrict__ cos_sin) {
  pdl_trigger();
  if (threadIdx.x == 0) FF_TL(status, KID_ROPE_KV, 0);
  pdl_wait();
  if (threadIdx.x == 0) FF_TL(status, KID_ROPE_KV, 1);
  const int vec_per_head = dim >> 4;                 // pairs of uint4
  const int heads = hq + 2 * hkv;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)rows * heads * vec_per_head;
  if (gid >= total) return;
  const int c = (int)(gid % vec_per_head);
  const int head = (int)((gid / vec_per_head) % heads);
  const int row = (int)(gid / ((long long)vec_per_head * heads));
  __nv_bfloat16* base = qkv + (size_t)row * ldqkv + (size_t)head * dim;
  const int half = dim >> 1;
  uint4 lo = reinterpret_cast<uint4*>(base)[c];
  uint4 hi = reinterpret_cast<uint4*>(base + half)[c];
  const bool is_v = head >= hq + hkv;
  if (!is_v) {
    const int pos = cos_sin ? 0 : positions[row];
    uint32_t* lp = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* hp = reinterpret_cast<uint32_t*>(&hi);
    const int rhalf = rot_dim >> 1;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf16x2(lp[j]), b = unpack_bf16x2(hp[j]);
      float ao[2] = {a.x, a.y}, bo[2] = {b.x, b.y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = c * 8 + j * 2 + e;               // index inside the half
        if (i < rhalf) {
          float sn, cs;
          if (cos_sin) {                                // per-row table (2-D / multi-axis rotary): already BF16-rounded
            const float2 t = cos_sin[(size_t)row * rhalf + i];
            cs = t.x; sn = t.y;
          } else {
            const float inv = inv_freq_tab ? inv_freq_tab[i] : 1.0f / powf(theta, (float)(2 * i) / (float)rot_dim);
            sincosf((float)pos * inv, &sn, &cs);
            cs = bf16r(cs); sn = bf16r(sn);             // cos/sin rounded to BF16
          }
          const float x1 = ao[e], x2 = bo[e];
          // BF16 arithmetic: every product and the final sum/difference round to BF16
          ao[e] = bf16r(bf16r(x1 * cs) - bf16r(x2 * sn));
          bo[e] = bf16r(bf16r(x2 * cs) + bf16r(x1 * sn));
        }
      }
      lp[j] = pack_bf16x2(ao[0], ao[1]);
      hp[j] = pack_bf16x2(bo[0], bo[1]);
    }
    reinterpret_cast<uint4*>(base)[c] = lo;
    reinterpret_cast<uint4*>(base + half)[c] = hi;
  }
  if (head >= hq) {
    const int slot = slots[row];
    if (slot < 0) return;                               // padding row: nothing cached
    const int blk = slot / block_size, off = slot - blk * block_size;
    if (blk >= num_blocks) { set_status(status, KID_ROPE_KV, FF_ERR_BOUNDS, row, slot); return; }
    const int kvh = is_v ? head - hq - hkv : head - hq;
    if (c == 0) dbg_write_once(status, KID_ROPE_KV, is_v ? DBG_KV_V : DBG_KV_K, (long long)slot * hkv + kvh);
    FF_DBG_CHECK(off >= 0 && off < block_size && kvh >= 0 && kvh < hkv, status, KID_ROPE_KV, row, kvh);
    __nv_bfloat16* dst = (is_v ? vcache : kcache) + (((size_t)blk * hkv + kvh) * block_size + off) * dim;
    reinterpret_cast<uint4*>(dst)[c] = lo;
    reinterpret_cast<uint4*>(dst + half)[c] = hi;
  }
}

// mode 0: bf16(silu(g)) * u rounded again   mode 1: single rounding
// mode 2: tanh-GELU(g) twice rounded         mode 4: clamped (DeepSeek) form in FP32, limit given
__device__ __forceinline__ float act_combine(float g, float u, int mode, float limit) {
  if (mode == 0) return bf16r(g / (1.f + __expf(-g))) * u;
  if (mode == 1) return (g / (1.f + __expf(-g))) * u;
  if (mode == 2) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    const float t = tanhf(k0 * (g + k1 * g * g * g));
    return bf16r(0.5f * g * (1.f + t)) * u;
  }
  // clamped: gate <= limit, up in [-limit, limit]
  g = fminf(g, limit); u = fmaxf(fminf(u, limit), -limit);
  return (g / (1.f + __expf(-g))) * u;
}

// (cos, sin) of position * inv_freq for every row and rotary pair, rounded to BF16 like the rotation
// kernels round them: computed once per step, read by every layer's fused QKV epilogue.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq_tab,
                                  float2* __restrict__ out, int rows, int rhalf, int rot_dim, float theta) {
  pdl_trigger();
  pdl_wait();
  const int gid = blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= rows * rhalf) return;
  const int row = gid / rhalf, i = gid - row * rhalf;
  const float inv = inv_freq_tab ? inv_freq_tab[i] : 1.0f / powf(theta, (float)(2 * i) / (float)rot_dim);
  float sn, cs;
  sincosf((float)positions[row] * inv, &sn, &cs);
  out[gid] = make_float2(bf16r(cs), bf16r(sn));
}

// interleaved != 0: gate/up alternate per 64 columns ([g0..g63 | u0..u63 | g64.. ]), the layout
// produced by a weight fused for the GEMM's SwiGLU epilogue; otherwise [gate | up] halves.
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int rows,
                                int f, int ldgu, int ldo, int mode, float limit, int interleaved) {
  pdl_trigger();
  pdl_wait();
  const int vec_per_row = f >> 3;
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (long long)rows * vec_per_row) return;
  const int row = (int)(gid / vec_per_row), c = (int)(gid % vec_per_row);
  const int gc = interleaved ? ((c >> 3) * 16 + (c & 7)) : c;           // 8 vectors per 64 columns
  const int uc = interleaved ? gc + 8 : c + vec_per_row;
  const uint4 g = reinterpret_cast<const uint4*>(gu + (size_t)row * ldgu)[gc];
  const uint4 u = reinterpret_cast<const uint4*>(gu + (size_t)row * ldgu)[uc];
  const uint32_t* gp = reinterpret_cast<const uint32_t*>(&g);
  const uint32_t* up = reinterpret_cast<const uint32_t*>(&u);
  uint4 o; uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 a = unpack_bf16x2(gp[j]), b = unpack_bf16x2(up[j]);
    op[j] = pack_bf16x2(act_combine(a.x, b.x, mode, limit), act_combine(a.y, b.y, mode, limit));
  }
  reinterpret_cast<uint4*>(out + (size_t)row * ldo)[c] = o;
}

// logits softcap: x = cap * tanh(x / cap) (Gemma), in place
__global__ void softcap_kernel(__nv_bfloat16* __restrict__ x, long long n, float cap) {
  pdl_trigger();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = __float2bfloat16(cap * tanhf(__bfloat162float(x[i]) / cap));
}

// ---------------------------------------------------------------------------------------
// argmax per row; ties -> lower index. valid_rows (device int, may be null) gates rows.
// ---------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const T* __restrict__ logits, int* __restrict__ out_ids, float* __restrict__ out_vals, int vocab,
                   int ld, int id_offset, const int* __restrict__ valid_rows, int* status) {
  pdl_trigger();
  if (threadIdx.x == 0) FF_TL(status, KID_SAMPLE, 0);
  pdl_wait();
  if (threadIdx.x == 0) FF_TL(status, KID_SAMPLE, 1);
  const int row = blockIdx.x;
  if (valid_rows && row >= *valid_rows) return;
  __shared__ float sv[32];
  __shared__ int si[32];
  float best = -INFINITY; int bi = 0x7fffffff;
  bool nonfinite = false;
  const T* p = logits + (size_t)row * ld;
  int i0 = 0;
  if (sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    // 16-byte vectors, two in flight per thread: a row of 128 K logits is 256 KB read by one CTA
    const int nvec = vocab >> 3;
    const uint4* pv = reinterpret_cast<const uint4*>(p);
    for (int i = threadIdx.x; i < nvec; i += 2 * blockDim.x) {
      uint4 u[2];
      u[0] = pv[i];
      const bool second = i + blockDim.x < nvec;
      u[1] = second ? pv[i + blockDim.x] : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1 && !second) break;
        const uint32_t* w = reinterpret_cast<const uint32_t*>(&u[h]);
        const int base = (i + h * blockDim.x) * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(w[j]);
          if (!(fabsf(f.x) <= 3.4e38f) || !(fabsf(f.y) <= 3.4e38f)) nonfinite = true;
          if (f.x > best || (f.x == best && base + 2 * j < bi)) { best = f.x; bi = base + 2 * j; }
          if (f.y > best || (f.y == best && base + 2 * j + 1 < bi)) { best = f.y; bi = base + 2 * j + 1; }
        }
      }
    }
    i0 = nvec << 3;
  }
  for (int i = i0 + threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = to_f<T>(p[i]);
    if (!(fabsf(v) <= 3.4e38f)) nonfinite = true;
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  if (nonfinite) set_status(status, KID_SAMPLE, FF_ERR_NONFINITE, row, 0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? sv[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      out_ids[row] = (bi == 0x7fffffff ? 0 : bi) + id_offset;
      if (out_vals) out_vals[row] = best;
    }
  }
}

// merge vocab-parallel candidates: vals/ids [ranks][rows] -> ids[rows]; ties -> lower id
__global__ void argmax_merge_kernel(const float* __restrict__ vals, const int* __restrict__ ids, int* __restrict__ out,
                                    int ranks, int rows) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float best = -INFINITY; int bi = 0x7fffffff;
  for (int k = 0; k < ranks; ++k) {
    const float v = vals[(size_t)k * rows + r]; const int i = ids[(size_t)k * rows + r];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  out[r] = bi;
}

// ---------------------------------------------------------------------------------------
// Philox4x32-10 and the stochastic sampler (one block per row).
// ---------------------------------------------------------------------------------------
__host__ __device__ inline void philox4x32_10(uint32_t key0, uint32_t key1, uint32_t c0, uint32_t c1, uint32_t c2,
                                              uint32_t c3, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)M0 * c0, p1 = (uint64_t)M1 * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ key0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ key1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    key0 += W0; key1 += W1;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__global__ void philox_uniform_kernel(float* __restrict__ out, long long n, unsigned long long seed,
                                      unsigned long long offset) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i * 4 >= n) return;
  uint32_t r[4];
  const unsigned long long ctr = offset + (unsigned long long)i;
  philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)ctr, (uint32_t)(ctr >> 32), 0, 0, r);
  for (int j = 0; j < 4; ++j)
    if (i * 4 + j < n) out[i * 4 + j] = ((r[j] >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

// Sampler: probabilities = softmax(penalised logits / temperature) restricted to top-k then
// top-p (smallest prefix of the descending order whose mass reaches top_p), renormalised;
// draws with one Philox uniform per row. Selection by iterative threshold search on the
// probability value, so no full sort is needed. history (may be null): [rows, hist_len] ids
// for the repetition penalty (logit > 0 ? /pen : *pen), -1 entries ignored.
__global__ void __launch_bounds__(1024)
sample_rows_kernel(const float* __restrict__ logits, int* __restrict__ out_ids, float* __restrict__ work, int vocab,
                   float temperature, int top_k, float top_p, float rep_penalty, const int* __restrict__ history,
                   int hist_len, unsigned long long seed, unsigned long long step) {
  const int row = blockIdx.x;
  const float* lg = logits + (size_t)row * vocab;
  float* pr = work + (size_t)row * vocab;
  __shared__ float red[32];
  __shared__ float s_val;
  __shared__ int s_cnt;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  // 1. penalised, temperature-scaled logits -> pr ; row max
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { pr[i] = lg[i]; }
  __syncthreads();
  if (history && rep_penalty != 1.0f) {
    for (int h = threadIdx.x; h < hist_len; h += blockDim.x) {
      const int id = history[(size_t)row * hist_len + h];
      if (id >= 0 && id < vocab) {
        // several history entries may name the same id; the write is idempotent because it is
        // computed from the unpenalised logit
        const float v = lg[id];
        pr[id] = v > 0.f ? v / rep_penalty : v * rep_penalty;
      }
    }
    __syncthreads();
  }
  const float inv_t = 1.0f / temperature;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float v = pr[i] * inv_t; pr[i] = v; mx = fmaxf(mx, v); }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = lane < nw ? red[lane] : -INFINITY; mx = warp_max(mx);
  __syncthreads();
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float e = __expf(pr[i] - mx); pr[i] = e; sum += e; }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = lane < nw ? red[lane] : 0.f; sum = warp_sum(sum);
  __syncthreads();
  const float inv_sum = 1.0f / sum;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) pr[i] *= inv_sum;
  __syncthreads();
  // 2. threshold search. Kept set = {p >= thr} for the LARGEST thr such that the set's mass
  //    reaches top_p or its size reaches top_k (mass measured on the full distribution).
  float lo = 0.f, hi = 1.0f;
  const int k = top_k > 0 && top_k < vocab ? top_k : vocab;
  for (int iter = 0; iter < 30; ++iter) {
    const float mid = 0.5f * (lo + hi);
    int cnt = 0; float mass = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float p = pr[i]; if (p >= mid) { cnt++; mass += p; } }
    mass = warp_sum(mass);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (threadIdx.x == 0) s_cnt = 0;
    if (lane == 0) red[warp] = mass;
    __syncthreads();
    if (lane == 0) atomicAdd(&s_cnt, cnt);
    float tm = lane < nw ? red[lane] : 0.f; tm = warp_sum(tm);
    __syncthreads();
    const int tc = s_cnt;
    if (tm >= top_p || tc >= k) lo = mid; else hi = mid;
    __syncthreads();
  }
  const float thr = lo;
  // 3. renormalise over kept set and draw
  float kept = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const float p = pr[i]; if (p >= thr) kept += p; }
  kept = warp_sum(kept);
  if (lane == 0) red[warp] = kept;
  __syncthreads();
  kept = lane < nw ? red[lane] : 0.f; kept = warp_sum(kept);
  if (threadIdx.x == 0) {
    uint32_t r[4];
    philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), (uint32_t)step, (uint32_t)(step >> 32), (uint32_t)row, 0, r);
    const float u = ((r[0] >> 8) + 0.5f) * (1.0f / 16777216.0f);
    s_val = u * kept;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // serial inverse-CDF over the kept set in id order (deterministic); vocab-length scan by
    // one thread is fine for sampling rows (not on the greedy hot path)
    const float target = s_val;
    float acc = 0.f; int pick = -1, last = 0;
    for (int i = 0; i < vocab; ++i) {
      const float p = pr[i];
      if (p >= thr) { acc += p; last = i; if (acc >= target) { pick = i; break; } }
    }
    out_ids[row] = pick >= 0 ? pick : last;
  }
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_rope_kv_paged(void* qkv, const int* positions, const int* slots, void* kcache, void* vcache,
                               const float* inv_freq, int rows, int hq, int hkv, int dim, int rot_dim, int block_size,
                               int num_blocks, float theta, int ldqkv, int* status, cudaStream_t s) {
  if (rows <= 0 || dim % 16 || rot_dim > dim || rot_dim % 2 || ldqkv % 8) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)rows * (hq + 2 * hkv) * (dim / 16);
  if (int lr_ = launch_pdl(rope_kv_paged_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, (__nv_bfloat16*)qkv, positions, slots,
      (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, inv_freq, rows, hq, hkv, dim, rot_dim, block_size, num_blocks,
      theta, ldqkv, status, (const float2*)nullptr)) return lr_;
  return launch_result();
}

// Same with the angles given as a table: cos_sin [rows, rot_dim/2] (cos, sin) FP32 holding BF16-rounded values.
// Serves rotary schemes whose angle is not position * inv_freq[i]: 2-D (row, column) rotary of vision towers and
// multi-axis rotary of vision-language decoders. slots / caches may be null (rotation only, hkv = 0).
FF_EXPORT int ff_rope_kv_paged_table(void* qkv, const float* cos_sin, const int* slots, void* kcache, void* vcache,
                                     int rows, int hq, int hkv, int dim, int rot_dim, int block_size, int num_blocks,
                                     int ldqkv, int* status, cudaStream_t s) {
  if (rows <= 0 || dim % 16 || rot_dim > dim || rot_dim % 2 || ldqkv % 8 || !cos_sin) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)rows * (hq + 2 * hkv) * (dim / 16);
  if (int lr_ = launch_pdl(rope_kv_paged_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, (__nv_bfloat16*)qkv,
      (const int*)nullptr, slots, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, (const float*)nullptr, rows, hq, hkv, dim,
      rot_dim, block_size, num_blocks, 1.0f, ldqkv, status, reinterpret_cast<const float2*>(cos_sin))) return lr_;
  return launch_result();
}

// out: float2 [rows, rot_dim/2]
FF_EXPORT int ff_rope_table(const int* positions, const float* inv_freq, float* out, int rows, int rot_dim, float theta,
                            cudaStream_t s) {
  if (rows <= 0 || rot_dim <= 0 || rot_dim % 2) return FF_HOST_BAD_SHAPE;
  const int rhalf = rot_dim / 2, total = rows * rhalf;
  if (int lr_ = launch_pdl(rope_table_kernel, dim3((total + 127) / 128), dim3(128), 0, s, 0, positions, inv_freq,
                           reinterpret_cast<float2*>(out), rows, rhalf, rot_dim, theta)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_silu_mul(const void* gu, void* out, int rows, int f, int ldgu, int ldo, int mode, float limit,
                          int interleaved, cudaStream_t s) {
  if (rows <= 0 || f <= 0 || f % 8 || ldgu % 8 || ldo % 8) return FF_HOST_BAD_SHAPE;
  if (interleaved && f % 64) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)rows * (f / 8);
  if (int lr_ = launch_pdl(silu_mul_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows,
                                                                   f, ldgu, ldo, mode, limit, interleaved)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_softcap(void* x, long long n, float cap, cudaStream_t s) {
  if (n <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr_ = launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, 0, (__nv_bfloat16*)x, n, cap)) return lr_;
  return launch_result();
}

// dtype: 0 = bf16 logits, 1 = fp32 logits
FF_EXPORT int ff_argmax_rows(const void* logits, int* out_ids, float* out_vals, int rows, int vocab, int ld, int dtype,
                             int id_offset, const int* valid_rows, int* status, cudaStream_t s) {
  if (rows <= 0 || vocab <= 0) return FF_HOST_BAD_SHAPE;
  int lr;
  if (dtype == 0) {
    lr = launch_pdl(argmax_rows_kernel<__nv_bfloat16>, dim3(rows), dim3(1024), 0, s, 0, (const __nv_bfloat16*)logits, out_ids,
                    out_vals, vocab, ld, id_offset, valid_rows, status);
  } else {
    lr = launch_pdl(argmax_rows_kernel<float>, dim3(rows), dim3(1024), 0, s, 0, (const float*)logits, out_ids, out_vals, vocab,
                    ld, id_offset, valid_rows, status);
  }
  if (lr) return lr;
  return launch_result();
}

FF_EXPORT int ff_argmax_merge(const float* vals, const int* ids, int* out, int ranks, int rows, cudaStream_t s) {
  if (ranks <= 0 || rows <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr_ = launch_pdl(argmax_merge_kernel, dim3((rows + 127) / 128), dim3(128), 0, s, 0, vals, ids, out, ranks, rows)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_philox_uniform(float* out, long long n, unsigned long long seed, unsigned long long offset,
                                cudaStream_t s) {
  if (n <= 0) return FF_HOST_BAD_SHAPE;
  const long long threads = (n + 3) / 4;
  philox_uniform_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(out, n, seed, offset);
  return launch_result();
}

// work: fp32 [rows, vocab] scratch for probabilities (caller-provided)
FF_EXPORT int ff_sample_rows(const float* logits, int* out_ids, float* work, int rows, int vocab, float temperature,
                             int top_k, float top_p, float rep_penalty, const int* history, int hist_len,
                             unsigned long long seed, unsigned long long step, cudaStream_t s) {
  if (rows <= 0 || vocab <= 0 || !(temperature > 0.f) || !(top_p > 0.f)) return FF_HOST_BAD_SHAPE;
  sample_rows_kernel<<<rows, 1024, 0, s>>>(logits, out_ids, work, vocab, temperature, top_k, top_p, rep_penalty,
                                           history, hist_len, seed, step);
  return launch_result();
}
