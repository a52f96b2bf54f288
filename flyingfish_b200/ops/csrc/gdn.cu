// Gated DeltaNet (linear-attention layers of hybrid models): O(1) state per sequence and head.
//   conv     : depthwise causal conv1d, 4 taps, no bias, over the fused q|k|v channels; the conv result is
//              rounded to BF16, SiLU applied, rounded to BF16; a 3-value history per channel carries the
//              previous rows across calls.
//   prep     : FP32 L2 normalisation of q and k per head, q scaled by 1/sqrt(dk); k heads expand to value
//              heads (value head h reads key head h / (heads / kheads)).
//   recurrent: per sequence and value head, for its rows in order
//                 S = S * exp(g);  kv = k^T S;  delta = (v - kv) * beta;  S += k (x) delta;  o = q^T S
//              (S_t = exp(g_t)(I - beta_t k_t k_t^T) S_{t-1} + beta_t k_t v_t^T), all state math FP32.
// Restates kernels/gdn/ of the reference (gdn_conv.cu:1-8, gdn_prep.cu:1-4, gdn_recurrent.cuh:1-16). There a
// block of 512 threads owns one head with the state in shared/global memory per step and prefill uses a chunked
// WY form; here one thread owns one column S[:, j] of the 128 x 128 state in registers for ALL rows of the
// sequence, so decode (one row) and prefill (many rows) are the same kernel and the state is read and written
// once per call.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int GDN_D = 128;           // dk = dv = 128

__device__ __forceinline__ float gdn_bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// x [rows, channels] bf16 rows of ONE sequence in order; weight [channels, 4] bf16; history [channels, 3] f32
// (x[r-3], x[r-2], x[r-1] before the first row), updated in place when commit != 0. out [rows, channels] bf16.
__global__ void gdn_conv_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                                float* __restrict__ history, __nv_bfloat16* __restrict__ out, int rows, int channels,
                                int commit) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  float w[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) w[t] = __bfloat162float(weight[c * 4 + t]);
  float h0 = history[c * 3], h1 = history[c * 3 + 1], h2 = history[c * 3 + 2];
  for (int r = 0; r < rows; ++r) {
    const float cur = __bfloat162float(x[(size_t)r * channels + c]);
    float acc = 0.f;
    acc = fmaf(w[0], h0, acc); acc = fmaf(w[1], h1, acc); acc = fmaf(w[2], h2, acc); acc = fmaf(w[3], cur, acc);
    const float y = gdn_bf16r(acc);
    out[(size_t)r * channels + c] = __float2bfloat16_rn(y / (1.0f + expf(-y)));
    h0 = h1; h1 = h2; h2 = cur;
  }
  if (commit) { history[c * 3] = h0; history[c * 3 + 1] = h1; history[c * 3 + 2] = h2; }
}

// Batched form: sequence s owns rows row_start[s] .. row_start[s+1] of x (row pitch ldx elements) and the history
// slab history[slot[s]] ([channels, 3] f32 each). grid (channel blocks, sequences).
__global__ void gdn_conv_batched_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ weight,
                                        float* __restrict__ history, __nv_bfloat16* __restrict__ out,
                                        const int* __restrict__ row_start, const int* __restrict__ slot, int channels,
                                        int ldx, int commit) {
  pdl_trigger();
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x, s = blockIdx.y;
  if (c >= channels) return;
  float w[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) w[t] = __bfloat162float(weight[c * 4 + t]);
  float* hist = history + ((size_t)slot[s] * channels + c) * 3;
  float h0 = hist[0], h1 = hist[1], h2 = hist[2];
  for (int r = row_start[s]; r < row_start[s + 1]; ++r) {
    const float cur = __bfloat162float(x[(size_t)r * ldx + c]);
    float acc = 0.f;
    acc = fmaf(w[0], h0, acc); acc = fmaf(w[1], h1, acc); acc = fmaf(w[2], h2, acc); acc = fmaf(w[3], cur, acc);
    const float y = gdn_bf16r(acc);
    out[(size_t)r * channels + c] = __float2bfloat16_rn(y / (1.0f + expf(-y)));
    h0 = h1; h1 = h2; h2 = cur;
  }
  if (commit) { hist[0] = h0; hist[1] = h1; hist[2] = h2; }
}

// conv_out [rows, (2*kheads + heads) * 128] bf16 = q | k | v ; q,k have kheads heads. Writes FP32 q, k
// [rows, heads, 128] (expanded to value heads, normalised, q scaled) and v [rows, heads, 128].
__global__ void gdn_prep_kernel(const __nv_bfloat16* __restrict__ conv_out, float* __restrict__ q, float* __restrict__ k,
                                float* __restrict__ v, int heads, int kheads, float eps) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y, h = blockIdx.x, lane = threadIdx.x;      // 32 threads, 4 dims each
  const int kh = h / (heads / kheads);
  const size_t ld = (size_t)(2 * kheads + heads) * GDN_D;
  const __nv_bfloat16* row = conv_out + (size_t)r * ld;
  float qv[4], kv[4], qs = 0.f, ks = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    qv[j] = __bfloat162float(row[(size_t)kh * GDN_D + lane * 4 + j]);
    kv[j] = __bfloat162float(row[(size_t)(kheads + kh) * GDN_D + lane * 4 + j]);
    qs += qv[j] * qv[j]; ks += kv[j] * kv[j];
  }
  qs = warp_sum(qs); ks = warp_sum(ks);
  const float qn = rsqrtf(qs + eps) * 0.08838834764831845f, kn = rsqrtf(ks + eps);     // 1/sqrt(128)
  const size_t o = ((size_t)r * heads + h) * GDN_D + lane * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    q[o + j] = qv[j] * qn; k[o + j] = kv[j] * kn;
    v[o + j] = __bfloat162float(row[(size_t)(2 * kheads + h) * GDN_D + lane * 4 + j]);
  }
}

// q, k, v [rows, heads, 128] f32, beta, g [rows, heads] f32, S [sequences, heads, 128(dk), 128(dv)] f32, out
// [rows, heads, 128] bf16. Sequence s owns rows row_start[s] .. row_start[s+1]. grid (heads, sequences), 128 threads.
__global__ void __launch_bounds__(128)
gdn_recurrent_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                     const float* __restrict__ beta, const float* __restrict__ g, float* __restrict__ S,
                     __nv_bfloat16* __restrict__ out, const int* __restrict__ row_start, int heads,
                     const int* __restrict__ state_slot) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sq[GDN_D], sk[GDN_D];
  const int h = blockIdx.x, s = blockIdx.y, j = threadIdx.x;
  const int ss = state_slot ? state_slot[s] : s;              // state slab of this sequence
  float* Sp = S + (((size_t)ss * heads + h) * GDN_D) * GDN_D + j;     // column j: element kk at Sp[kk * 128]
  float st[GDN_D];
#pragma unroll
  for (int kk = 0; kk < GDN_D; ++kk) st[kk] = Sp[(size_t)kk * GDN_D];
  for (int r = row_start[s]; r < row_start[s + 1]; ++r) {
    const size_t o = ((size_t)r * heads + h) * GDN_D;
    __syncthreads();
    sq[j] = q[o + j]; sk[j] = k[o + j];
    __syncthreads();
    const float decay = expf(g[(size_t)r * heads + h]), b = beta[(size_t)r * heads + h];
    float kvj = 0.f;
#pragma unroll
    for (int kk = 0; kk < GDN_D; ++kk) { st[kk] *= decay; kvj = fmaf(sk[kk], st[kk], kvj); }
    const float delta = (v[o + j] - kvj) * b;
    float oj = 0.f;
#pragma unroll
    for (int kk = 0; kk < GDN_D; ++kk) { st[kk] = fmaf(sk[kk], delta, st[kk]); oj = fmaf(sq[kk], st[kk], oj); }
    out[o + j] = __float2bfloat16_rn(oj);
  }
#pragma unroll
  for (int kk = 0; kk < GDN_D; ++kk) Sp[(size_t)kk * GDN_D] = st[kk];
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_gdn_conv(const void* x, const void* weight, float* history, void* out, int rows, int channels, int commit,
                          cudaStream_t s) {
  if (rows <= 0 || channels <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(gdn_conv_kernel, dim3((channels + 255) / 256), dim3(256), 0, s, 0, (const __nv_bfloat16*)x,
                          (const __nv_bfloat16*)weight, history, (__nv_bfloat16*)out, rows, channels, commit)) return lr;
  return launch_result();
}

FF_EXPORT int ff_gdn_prep(const void* conv_out, float* q, float* k, float* v, int rows, int heads, int kheads, float eps,
                          cudaStream_t s) {
  if (rows <= 0 || heads <= 0 || kheads <= 0 || heads % kheads) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(gdn_prep_kernel, dim3(heads, rows), dim3(32), 0, s, 0, (const __nv_bfloat16*)conv_out, q, k, v, heads,
                          kheads, eps)) return lr;
  return launch_result();
}

FF_EXPORT int ff_gdn_recurrent(const float* q, const float* k, const float* v, const float* beta, const float* g, float* S,
                               void* out, const int* row_start, int sequences, int heads, cudaStream_t s) {
  if (sequences <= 0 || heads <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(gdn_recurrent_kernel, dim3(heads, sequences), dim3(128), 0, s, 0, q, k, v, beta, g, S,
                          (__nv_bfloat16*)out, row_start, heads, (const int*)nullptr)) return lr;
  return launch_result();
}

// Batched forms for a model's forward: sequences address their state through slot indices.
FF_EXPORT int ff_gdn_recurrent_slots(const float* q, const float* k, const float* v, const float* beta, const float* g,
                                     float* S, void* out, const int* row_start, const int* state_slot, int sequences,
                                     int heads, cudaStream_t s) {
  if (sequences <= 0 || heads <= 0 || !state_slot) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(gdn_recurrent_kernel, dim3(heads, sequences), dim3(128), 0, s, 0, q, k, v, beta, g, S,
                          (__nv_bfloat16*)out, row_start, heads, state_slot)) return lr;
  return launch_result();
}

FF_EXPORT int ff_gdn_conv_batched(const void* x, const void* weight, float* history, void* out, const int* row_start,
                                  const int* slot, int sequences, int channels, int ldx, int commit, cudaStream_t s) {
  if (sequences <= 0 || channels <= 0 || ldx < channels) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(gdn_conv_batched_kernel, dim3((channels + 255) / 256, sequences), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)x, (const __nv_bfloat16*)weight, history, (__nv_bfloat16*)out, row_start,
                          slot, channels, ldx, commit)) return lr;
  return launch_result();
}
