// Speech-model kernels (FastConformer encoders with a transducer decoder):
//   logmel_frames      : pre-emphasis + centred Hann window + radix-2 FFT in shared memory + power spectrum +
//                        mel filterbank + log, one CTA per frame (src/audio.rs:204-300 of the reference is the host
//                        loop this replaces)
//   feat_normalize     : per-(utterance, mel band) mean / unbiased standard deviation over the valid frames
//   sub_conv_first     : 3x3 stride-2 convolution of the one-channel mel image into C channels + ReLU, channels-last
//   sub_dwconv         : 3x3 stride-2 depthwise convolution, channels-last, input rows beyond the valid length read as 0
//   glu_dwconv1d       : the conformer convolution module between its two pointwise GEMMs in one pass:
//                        bias + GLU + time mask + depthwise conv over time + (batch-norm folded) bias + SiLU
//   scale_add_layernorm: h += scale * (delta + bias); y = LayerNorm(h)  (macaron residuals and the norm that follows)
//   relpos_attention   : Transformer-XL relative-position attention, flash style on mma.sync: the content term
//                        (q+u)K^T and the position term (q+v)P^T are both tensor-core tiles; the position tile of a
//                        16-query warp is computed for the 79 relative offsets its 16 x 64 score tile touches and
//                        read back skewed through shared memory (kernels/speech_ops.cu "relative attention")
//   lstm_cell / tdt_*  : prediction-network cell, joint input and the greedy token-and-duration selection with the
//                        decode state (frame, token, trajectory) kept on the device, so that a decode step is a
//                        fixed launch sequence replayed from a CUDA graph without a host read per step
//                        (src/backend/cuda/engine_parakeet.rs:2550-2633 reads the selection back every step)
#include "ptx.cuh"
#include "host_util.h"
#include "mma_sync.cuh"

namespace ff {

__device__ __forceinline__ float bfr_s(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------------------
// log-mel front end
// ------------------------------------------------------------------------------------------------
constexpr int MEL_MAX_FFT = 1024;

// grid (frames, batch), 256 threads. wave: [batch, max_samples] FP32, lens: samples per utterance.
// window: [n_fft] (already centred), filters: [mel_bins, n_fft/2+1], band_range: [mel_bins, 2] = first / end bin with a
// non-zero weight. out: [batch, frames, mel_bins] FP32; frames at or beyond lens / hop are written as zero.
__global__ void __launch_bounds__(256)
logmel_kernel(const float* __restrict__ wave, const int* __restrict__ lens, const float* __restrict__ window,
              const float* __restrict__ filters, const int* __restrict__ band_range, float* __restrict__ out,
              long long max_samples, int frames, int n_fft, int log2n, int hop, int mel_bins, float preemph,
              float log_guard) {
  __shared__ float s_re[MEL_MAX_FFT], s_im[MEL_MAX_FFT];
  __shared__ float s_twr[MEL_MAX_FFT / 2], s_twi[MEL_MAX_FFT / 2];
  const int t = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int len = lens[b], valid = len / hop;
  float* dst = out + ((size_t)b * frames + t) * mel_bins;
  if (t >= valid) {
    for (int m = tid; m < mel_bins; m += 256) dst[m] = 0.f;
    return;
  }
  const float* w = wave + (size_t)b * max_samples;
  const int half = n_fft >> 1;
  for (int i = tid; i < half; i += 256) {
    float sn, cs;
    sincospif(-2.0f * (float)i / (float)n_fft, &sn, &cs);
    s_twr[i] = cs; s_twi[i] = sn;
  }
  for (int i = tid; i < n_fft; i += 256) {
    const long long pos = (long long)t * hop + i - half;
    float v = 0.f;
    if (pos >= 0 && pos < len) v = pos == 0 ? w[0] : w[pos] - preemph * w[pos - 1];
    const int r = (int)(__brev((unsigned)i) >> (32 - log2n));
    s_re[r] = v * window[i];
    s_im[r] = 0.f;
  }
  __syncthreads();
  for (int s = 1; s <= log2n; ++s) {
    const int hs = 1 << (s - 1), tw_step = n_fft >> s;
    for (int i = tid; i < half; i += 256) {
      const int grp = i >> (s - 1), j = i & (hs - 1);
      const int a = (grp << s) + j, c = a + hs;
      const float wr = s_twr[j * tw_step], wi = s_twi[j * tw_step];
      const float xr = s_re[c], xi = s_im[c];
      const float tr = xr * wr - xi * wi, ti = xr * wi + xi * wr;
      const float ur = s_re[a], ui = s_im[a];
      s_re[a] = ur + tr; s_im[a] = ui + ti;
      s_re[c] = ur - tr; s_im[c] = ui - ti;
    }
    __syncthreads();
  }
  const int bins = half + 1;
  for (int i = tid; i < bins; i += 256) s_re[i] = s_re[i] * s_re[i] + s_im[i] * s_im[i];
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int m = warp; m < mel_bins; m += 8) {
    const int lo = band_range[2 * m], hi = band_range[2 * m + 1];
    const float* f = filters + (size_t)m * bins;
    float acc = 0.f;
    for (int i = lo + lane; i < hi; i += 32) acc = fmaf(f[i], s_re[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) dst[m] = logf(acc + log_guard);
  }
}

// grid (ceil(mel_bins / 32), batch), block (32, 8): in place, feat [batch, frames, mel_bins]
__global__ void feat_normalize_kernel(float* __restrict__ feat, const int* __restrict__ lens, int frames, int mel_bins,
                                      int hop, float eps) {
  __shared__ float s_red[8][33];
  const int m = blockIdx.x * 32 + threadIdx.x, b = blockIdx.y, ty = threadIdx.y;
  const int valid = min(lens[b] / hop, frames);
  float* base = feat + (size_t)b * frames * mel_bins;
  float sum = 0.f;
  if (m < mel_bins)
    for (int t = ty; t < valid; t += 8) sum += base[(size_t)t * mel_bins + m];
  s_red[ty][threadIdx.x] = sum;
  __syncthreads();
  float mean = 0.f;
  for (int i = 0; i < 8; ++i) mean += s_red[i][threadIdx.x];
  mean /= (float)max(valid, 1);
  __syncthreads();
  float sq = 0.f;
  if (m < mel_bins)
    for (int t = ty; t < valid; t += 8) { const float d = base[(size_t)t * mel_bins + m] - mean; sq = fmaf(d, d, sq); }
  s_red[ty][threadIdx.x] = sq;
  __syncthreads();
  float var = 0.f;
  for (int i = 0; i < 8; ++i) var += s_red[i][threadIdx.x];
  const float inv = 1.f / (sqrtf(var / (float)max(valid - 1, 1)) + eps);
  if (m < mel_bins)
    for (int t = ty; t < valid; t += 8) base[(size_t)t * mel_bins + m] = (base[(size_t)t * mel_bins + m] - mean) * inv;
}

// ------------------------------------------------------------------------------------------------
// sub-sampling stem, channels-last
// ------------------------------------------------------------------------------------------------
// in: [batch, T, F] FP32, w: [9, C] FP32 (tap-major), bias [C]; out: [batch, T1, F1, C] BF16 = relu(conv), zero for
// output rows at or beyond valid_out[b]. One thread per (pixel, 8 channels).
__global__ void __launch_bounds__(256)
sub_conv_first_kernel(const float* __restrict__ in, const float* __restrict__ w, const float* __restrict__ bias,
                      const int* __restrict__ valid_out, __nv_bfloat16* __restrict__ out, int T, int F, int T1, int F1,
                      int C, int pad_t, int pad_f, long long total) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  if (gid >= total) return;
  const int cv = C >> 3;
  const int c0 = (int)(gid % cv) * 8;
  long long pix = gid / cv;
  const int f1 = (int)(pix % F1); pix /= F1;
  const int t1 = (int)(pix % T1);
  const int b = (int)(pix / T1);
  uint4 o = make_uint4(0u, 0u, 0u, 0u);
  if (t1 < valid_out[b]) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bias[c0 + j];
#pragma unroll
    for (int dt = 0; dt < 3; ++dt) {
      const int t = 2 * t1 + dt - pad_t;
      if (t < 0 || t >= T) continue;
#pragma unroll
      for (int df = 0; df < 3; ++df) {
        const int f = 2 * f1 + df - pad_f;
        if (f < 0 || f >= F) continue;
        const float x = in[((size_t)b * T + t) * F + f];
        const float4 w0 = *reinterpret_cast<const float4*>(w + (size_t)(dt * 3 + df) * C + c0);
        const float4 w1 = *reinterpret_cast<const float4*>(w + (size_t)(dt * 3 + df) * C + c0 + 4);
        acc[0] = fmaf(x, w0.x, acc[0]); acc[1] = fmaf(x, w0.y, acc[1]); acc[2] = fmaf(x, w0.z, acc[2]);
        acc[3] = fmaf(x, w0.w, acc[3]); acc[4] = fmaf(x, w1.x, acc[4]); acc[5] = fmaf(x, w1.y, acc[5]);
        acc[6] = fmaf(x, w1.z, acc[6]); acc[7] = fmaf(x, w1.w, acc[7]);
      }
    }
    o.x = pack_bf16x2(fmaxf(acc[0], 0.f), fmaxf(acc[1], 0.f)); o.y = pack_bf16x2(fmaxf(acc[2], 0.f), fmaxf(acc[3], 0.f));
    o.z = pack_bf16x2(fmaxf(acc[4], 0.f), fmaxf(acc[5], 0.f)); o.w = pack_bf16x2(fmaxf(acc[6], 0.f), fmaxf(acc[7], 0.f));
  }
  *reinterpret_cast<uint4*>(out + (size_t)gid * 8) = o;
}

// in: [batch, T, F, C] BF16 (rows t >= valid_in[b] read as zero), w: [9, C] FP32, bias [C];
// out: [batch, T1, F1, C] BF16, no activation (a pointwise GEMM follows).
__global__ void __launch_bounds__(256)
sub_dwconv_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ w, const float* __restrict__ bias,
                  const int* __restrict__ valid_in, __nv_bfloat16* __restrict__ out, int T, int F, int T1, int F1, int C,
                  int pad_t, int pad_f, long long total) {
  pdl_trigger();
  pdl_wait();
  const long long gid = (long long)blockIdx.x * 256 + threadIdx.x;
  if (gid >= total) return;
  const int cv = C >> 3;
  const int c0 = (int)(gid % cv) * 8;
  long long pix = gid / cv;
  const int f1 = (int)(pix % F1); pix /= F1;
  const int t1 = (int)(pix % T1);
  const int b = (int)(pix / T1);
  const int vin = min(valid_in[b], T);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = bias[c0 + j];
#pragma unroll
  for (int dt = 0; dt < 3; ++dt) {
    const int t = 2 * t1 + dt - pad_t;
    if (t < 0 || t >= vin) continue;
#pragma unroll
    for (int df = 0; df < 3; ++df) {
      const int f = 2 * f1 + df - pad_f;
      if (f < 0 || f >= F) continue;
      const uint4 xv = *reinterpret_cast<const uint4*>(in + (((size_t)b * T + t) * F + f) * C + c0);
      const float4 w0 = *reinterpret_cast<const float4*>(w + (size_t)(dt * 3 + df) * C + c0);
      const float4 w1 = *reinterpret_cast<const float4*>(w + (size_t)(dt * 3 + df) * C + c0 + 4);
      const float2 x0 = unpack_bf16x2(xv.x), x1 = unpack_bf16x2(xv.y), x2 = unpack_bf16x2(xv.z), x3 = unpack_bf16x2(xv.w);
      acc[0] = fmaf(x0.x, w0.x, acc[0]); acc[1] = fmaf(x0.y, w0.y, acc[1]); acc[2] = fmaf(x1.x, w0.z, acc[2]);
      acc[3] = fmaf(x1.y, w0.w, acc[3]); acc[4] = fmaf(x2.x, w1.x, acc[4]); acc[5] = fmaf(x2.y, w1.y, acc[5]);
      acc[6] = fmaf(x3.x, w1.z, acc[6]); acc[7] = fmaf(x3.y, w1.w, acc[7]);
    }
  }
  uint4 o;
  o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
  o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + (size_t)gid * 8) = o;
}

// ------------------------------------------------------------------------------------------------
// conformer convolution module, middle part
// ------------------------------------------------------------------------------------------------
constexpr int DW_STRIP = 8, DW_MAX_K = 32;

// x: [batch * T, 2H] BF16 (value half then gate half), xbias: [2H] FP32 or null; w: [K, H] FP32, bias [H] FP32;
// y: [batch * T, H] BF16 = act(sum_k w[k] * glu(x)[t + k - left] + bias), glu rows outside [0, lens[b]) read as zero.
// grid (ceil(H / 2 / 128), ceil(T / DW_STRIP), batch): one thread per channel pair and strip of 8 frames; every input
// frame of the strip's window is read once and scattered into the outputs it feeds. KMAX bounds the unrolled taps.
template <int KMAX>
__global__ void __launch_bounds__(128)
glu_dwconv1d_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ xbias, const float* __restrict__ w,
                    const float* __restrict__ bias, const int* __restrict__ lens, __nv_bfloat16* __restrict__ y, int T,
                    int H, int K, int left, int silu) {
  pdl_trigger();
  pdl_wait();
  const int cp = blockIdx.x * 128 + threadIdx.x;
  if (cp * 2 >= H) return;
  const int c = cp * 2, t0 = blockIdx.y * DW_STRIP, b = blockIdx.z;
  const int len = min(lens[b], T);
  float2 wk[KMAX];
#pragma unroll
  for (int k = 0; k < KMAX; ++k) wk[k] = k < K ? *reinterpret_cast<const float2*>(w + (size_t)k * H + c) : make_float2(0.f, 0.f);
  float2 bv = make_float2(0.f, 0.f), bg = make_float2(0.f, 0.f);
  if (xbias) { bv = *reinterpret_cast<const float2*>(xbias + c); bg = *reinterpret_cast<const float2*>(xbias + H + c); }
  const float2 ob = *reinterpret_cast<const float2*>(bias + c);
  float2 acc[DW_STRIP];
#pragma unroll
  for (int i = 0; i < DW_STRIP; ++i) acc[i] = ob;
#pragma unroll
  for (int j = 0; j < DW_STRIP + KMAX - 1; ++j) {
    const int t = t0 + j - left;
    if (j < DW_STRIP + K - 1 && t >= 0 && t < len) {
      const __nv_bfloat16* row = x + ((size_t)b * T + t) * 2 * H;
      const float2 v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + c));
      const float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(row + H + c));
      float2 u;
      u.x = bfr_s((v.x + bv.x) * sigmoidf_(g.x + bg.x));
      u.y = bfr_s((v.y + bv.y) * sigmoidf_(g.y + bg.y));
#pragma unroll
      for (int i = 0; i < DW_STRIP; ++i) {
        if (j - i >= 0 && j - i < KMAX) {       // taps at or beyond K hold zero weights
          acc[i].x = fmaf(wk[j - i].x, u.x, acc[i].x);
          acc[i].y = fmaf(wk[j - i].y, u.y, acc[i].y);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < DW_STRIP; ++i) {
    const int t = t0 + i;
    if (t < T) {
      float2 o = acc[i];
      if (silu) { o.x = o.x * sigmoidf_(o.x); o.y = o.y * sigmoidf_(o.y); }
      *reinterpret_cast<uint32_t*>(y + ((size_t)b * T + t) * H + c) = pack_bf16x2(o.x, o.y);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// h += scale * (delta + dbias);  y = LayerNorm(h) * w + b      (h, delta, y BF16; dbias, w, b FP32)
// ------------------------------------------------------------------------------------------------
constexpr int SAL_MAX = 16;     // hidden <= 128 * 4 * 16 = 8192

__device__ __forceinline__ float block_sum_sp(float v, float* s_red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
  __syncthreads();
  return s_red[0] + s_red[1] + s_red[2] + s_red[3];
}

__global__ void __launch_bounds__(128)
scale_add_layernorm_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ delta,
                           const float* __restrict__ dbias, const float* __restrict__ w, const float* __restrict__ b,
                           __nv_bfloat16* __restrict__ y, int hidden, int ldh, int ldd, int ldy, float scale, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_red[4];
  const int row = blockIdx.x, nq = hidden >> 2;
  float v[SAL_MAX][4];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < SAL_MAX; ++i) {
    const int q = threadIdx.x + i * 128;
    if (q < nq) {
      const uint2 hv = *reinterpret_cast<const uint2*>(h + (size_t)row * ldh + q * 4);
      float2 a = unpack_bf16x2(hv.x), c = unpack_bf16x2(hv.y);
      if (delta) {
        const uint2 dv = *reinterpret_cast<const uint2*>(delta + (size_t)row * ldd + q * 4);
        float2 d0 = unpack_bf16x2(dv.x), d1 = unpack_bf16x2(dv.y);
        if (dbias) {
          const float4 db = *reinterpret_cast<const float4*>(dbias + q * 4);
          d0.x += db.x; d0.y += db.y; d1.x += db.z; d1.y += db.w;
        }
        a.x = bfr_s(fmaf(scale, d0.x, a.x)); a.y = bfr_s(fmaf(scale, d0.y, a.y));
        c.x = bfr_s(fmaf(scale, d1.x, c.x)); c.y = bfr_s(fmaf(scale, d1.y, c.y));
        uint2 o; o.x = pack_bf16x2(a.x, a.y); o.y = pack_bf16x2(c.x, c.y);
        *reinterpret_cast<uint2*>(h + (size_t)row * ldh + q * 4) = o;
      }
      v[i][0] = a.x; v[i][1] = a.y; v[i][2] = c.x; v[i][3] = c.y;
      sum += a.x + a.y + c.x + c.y;
    }
  }
  if (y == nullptr) return;
  const float mean = block_sum_sp(sum, s_red) / (float)hidden;
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < SAL_MAX; ++i) {
    const int q = threadIdx.x + i * 128;
    if (q < nq) {
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float d = v[i][j] - mean; sq = fmaf(d, d, sq); }
    }
  }
  const float rstd = rsqrtf(block_sum_sp(sq, s_red) / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < SAL_MAX; ++i) {
    const int q = threadIdx.x + i * 128;
    if (q < nq) {
      const float4 wv = *reinterpret_cast<const float4*>(w + q * 4);
      float4 bb = make_float4(0.f, 0.f, 0.f, 0.f);
      if (b) bb = *reinterpret_cast<const float4*>(b + q * 4);
      uint2 o;
      o.x = pack_bf16x2(fmaf((v[i][0] - mean) * rstd, wv.x, bb.x), fmaf((v[i][1] - mean) * rstd, wv.y, bb.y));
      o.y = pack_bf16x2(fmaf((v[i][2] - mean) * rstd, wv.z, bb.z), fmaf((v[i][3] - mean) * rstd, wv.w, bb.w));
      *reinterpret_cast<uint2*>(y + (size_t)row * ldy + q * 4) = o;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// relative-position attention
// ------------------------------------------------------------------------------------------------
// q, k, v: rows b * T + i, head h at column h * D (leading dimensions ldq / ldk / ldv); pos: [2T - 1, heads * D], row c
// holds the projected embedding of relative offset (T - 1 - c), so the score of query i and key j uses row
// T - 1 - i + j. bias_u / bias_v: [heads, D] FP32. Keys j >= lens[b], j < i - left or j > i + right are masked
// (left / right < 0: unlimited); with chunk > 0 left / right count chunks of `chunk` rows instead: query chunk c sees
// key chunks c - left .. c + right. out rows i >= lens[b] are zero.
// grid (ceil(T / 64), heads, batch), 128 threads: warp w owns query rows i0 + 16w .. +15; key tiles of 64.
constexpr int RA_Q = 64, RA_KEYS = 64, RA_WIN = 128, RA_RAW_LD = 81;

template <int D>
constexpr int ra_smem_bytes() { return (RA_Q + 2 * RA_KEYS + RA_WIN) * D * 2 + 4 * 16 * RA_RAW_LD * 4 + 2 * D * 4; }

template <int D>
__global__ void __launch_bounds__(128)
relpos_attention_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                        const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ pos,
                        const float* __restrict__ bias_u, const float* __restrict__ bias_v, const int* __restrict__ lens,
                        __nv_bfloat16* __restrict__ out, int T, int ldq, int ldk, int ldv, int ldp, int ldo, int left,
                        int right, int chunk, float scale_log2) {
  pdl_trigger();
  pdl_wait();
  constexpr int CH = D / 8;
  extern __shared__ __align__(128) uint8_t ra_smem[];
  uint8_t* sQ = ra_smem;
  uint8_t* sK = sQ + RA_Q * D * 2;
  uint8_t* sV = sK + RA_KEYS * D * 2;
  uint8_t* sP = sV + RA_KEYS * D * 2;
  float* sRaw = reinterpret_cast<float*>(sP + RA_WIN * D * 2);
  float* sU = sRaw + 4 * 16 * RA_RAW_LD;
  float* sVb = sU + D;
  const int i0 = blockIdx.x * RA_Q, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int len = min(lens[b], T);
  const size_t row0 = (size_t)b * T;
  for (int i = tid; i < RA_Q * CH; i += 128) {
    const int r = i / CH, c = i - r * CH;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (i0 + r < T) val = *reinterpret_cast<const uint4*>(q + (row0 + i0 + r) * ldq + (size_t)h * D + c * 8);
    *reinterpret_cast<uint4*>(sQ + ms_off(r, c, CH)) = val;
  }
  for (int i = tid; i < D; i += 128) { sU[i] = bias_u[(size_t)h * D + i]; sVb[i] = bias_v[(size_t)h * D + i]; }
  __syncthreads();
  const uint32_t sQa = smem_u32(sQ), sKa = smem_u32(sK), sVa = smem_u32(sV), sPa = smem_u32(sP);
  // A fragments of (q + u) and (q + v), rounded to BF16 once: 2 x D/16 x 4 registers
  uint32_t au[D / 16][4], av[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ms_ldsm4(sQa + ms_off(warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4), CH), a[0], a[1], a[2], a[3]);
    const int c0 = kk * 16 + 2 * t4;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int col = c0 + ((r >> 1) << 3);
      const float2 f = unpack_bf16x2(a[r]);
      au[kk][r] = pack_bf16x2(f.x + sU[col], f.y + sU[col + 1]);
      av[kk][r] = pack_bf16x2(f.x + sVb[col], f.y + sVb[col + 1]);
    }
  }
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-3.0e38f, -3.0e38f}, l_run[2] = {0.f, 0.f};
  float* raw = sRaw + warp * 16 * RA_RAW_LD;
  const int qi[2] = {i0 + warp * 16 + g, i0 + warp * 16 + g + 8};

  int j_begin = 0, j_end = len;
  if (chunk > 0) {
    // chunk-wise context: query chunk c sees key chunks c - left .. c + right (streaming encoders)
    j_begin = max(0, (i0 / chunk - left) * chunk) / RA_KEYS * RA_KEYS;
    j_end = min(len, ((i0 + RA_Q - 1) / chunk + right + 1) * chunk);
  } else {
    if (left >= 0) j_begin = max(0, i0 - left) / RA_KEYS * RA_KEYS;
    if (right >= 0) j_end = min(len, i0 + RA_Q + right);
  }
  for (int j0 = j_begin; j0 < j_end; j0 += RA_KEYS) {
    __syncthreads();                     // the previous tile's K, V and window are no longer read
    for (int i = tid; i < RA_KEYS * CH; i += 128) {
      const int r = i / CH, c = i - r * CH;
      uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = kv;
      if (j0 + r < len) {
        kv = *reinterpret_cast<const uint4*>(k + (row0 + j0 + r) * ldk + (size_t)h * D + c * 8);
        vv = *reinterpret_cast<const uint4*>(v + (row0 + j0 + r) * ldv + (size_t)h * D + c * 8);
      }
      *reinterpret_cast<uint4*>(sK + ms_off(r, c, CH)) = kv;
      *reinterpret_cast<uint4*>(sV + ms_off(r, c, CH)) = vv;
    }
    // window of relative rows: local row r <-> table row T - 1 - (i0 + 63) + j0 + r
    const int cbase = T - 1 - i0 - (RA_Q - 1) + j0;
    for (int i = tid; i < RA_WIN * CH; i += 128) {
      const int r = i / CH, c = i - r * CH;
      const int pr = cbase + r;
      uint4 pv = make_uint4(0u, 0u, 0u, 0u);
      if (pr >= 0 && pr < 2 * T - 1) pv = *reinterpret_cast<const uint4*>(pos + (size_t)pr * ldp + (size_t)h * D + c * 8);
      *reinterpret_cast<uint4*>(sP + ms_off(r, c, CH)) = pv;
    }
    __syncthreads();
    // content term: s[n][.] for keys j0 + 8n .. +7
    float s[RA_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < RA_KEYS / 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int n2 = 0; n2 < RA_KEYS / 16; ++n2) {
        uint32_t b0, b1, b2, b3;
        ms_ldsm4(sKa + ms_off(n2 * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1), CH), b0, b1, b2, b3);
        ms_mma(s[2 * n2], au[kk], b0, b1);
        ms_mma(s[2 * n2 + 1], au[kk], b2, b3);
      }
    }
    // position term over this warp's 80 window rows (local rows wb .. wb + 79), staged skewed through shared memory
    const int wb = (RA_Q - 16) - 16 * warp;
#pragma unroll
    for (int n2 = 0; n2 < 5; ++n2) {
      float r0[4] = {0.f, 0.f, 0.f, 0.f}, r1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t b0, b1, b2, b3;
        ms_ldsm4(sPa + ms_off(wb + n2 * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1), CH), b0, b1, b2, b3);
        ms_mma(r0, av[kk], b0, b1);
        ms_mma(r1, av[kk], b2, b3);
      }
      const int col = n2 * 16 + 2 * t4;
      raw[g * RA_RAW_LD + col] = r0[0]; raw[g * RA_RAW_LD + col + 1] = r0[1];
      raw[(g + 8) * RA_RAW_LD + col] = r0[2]; raw[(g + 8) * RA_RAW_LD + col + 1] = r0[3];
      raw[g * RA_RAW_LD + col + 8] = r1[0]; raw[g * RA_RAW_LD + col + 9] = r1[1];
      raw[(g + 8) * RA_RAW_LD + col + 8] = r1[2]; raw[(g + 8) * RA_RAW_LD + col + 9] = r1[3];
    }
    __syncwarp();
    // score(i, j) = content + raw[i_local][j_local + 15 - i_local]; mask; online soft-max
    float mx[2] = {-3.0e38f, -3.0e38f};
#pragma unroll
    for (int n = 0; n < RA_KEYS / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int rl = g + ((e >> 1) << 3), jl = n * 8 + 2 * t4 + (e & 1);
        const int i = qi[e >> 1], j = j0 + jl;
        float sc = (s[n][e] + raw[rl * RA_RAW_LD + jl + 15 - rl]) * scale_log2;
        bool ok = j < len;
        if (chunk > 0) { const int qc = i / chunk, kc = j / chunk; ok = ok && kc >= qc - left && kc <= qc + right; }
        else ok = ok && (left < 0 || j >= i - left) && (right < 0 || j <= i + right);
        sc = ok ? sc : -3.0e38f;
        s[n][e] = sc;
        mx[e >> 1] = fmaxf(mx[e >> 1], sc);
      }
    }
    __syncwarp();                         // raw is rewritten by the next tile
    float resc[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(m_run[r], mx[r]);
      resc[r] = exp2f(m_run[r] - mnew);
      m_run[r] = mnew;
      l_run[r] *= resc[r];
    }
    uint32_t pa[RA_KEYS / 16][4];
#pragma unroll
    for (int n = 0; n < RA_KEYS / 8; ++n) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        // a fully masked element stays exactly zero even while the running maximum is still the initial value
        p[e] = s[n][e] <= -1.0e38f ? 0.f : exp2f(s[n][e] - m_run[e >> 1]);
        p[e] = bfr_s(p[e]);
        l_run[e >> 1] += p[e];
      }
      pa[n >> 1][(n & 1) * 2] = pack_bf16x2(p[0], p[1]);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(p[2], p[3]);
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= resc[0]; o[i][1] *= resc[0]; o[i][2] *= resc[1]; o[i][3] *= resc[1]; }
#pragma unroll
    for (int ks = 0; ks < RA_KEYS / 16; ++ks) {
      const int key = ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t b0, b1, b2, b3;
        ms_ldsm4t(sVa + ms_off(key, dp * 2 + (lane >> 4), CH), b0, b1, b2, b3);
        ms_mma(o[2 * dp], pa[ks], b0, b1);
        ms_mma(o[2 * dp + 1], pa[ks], b2, b3);
      }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = qi[r];
    if (i >= T) continue;
    const float inv = (i < len && l_run[r] > 0.f) ? 1.f / l_run[r] : 0.f;
    __nv_bfloat16* dst = out + (row0 + i) * ldo + (size_t)h * D;
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
      *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t4) = pack_bf16x2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
  }
}

// ------------------------------------------------------------------------------------------------
// transducer decoder
// ------------------------------------------------------------------------------------------------
// decode state words
// (TS_VALID = encoder rows of the utterance, TS_CAP = trajectory entries allowed, TS_MAXSYM = tokens one frame may emit:
// set by the host per utterance; TS_SYMS = tokens emitted at the current frame so far)
enum { TS_FRAME = 0, TS_TOKEN = 1, TS_COUNT = 2, TS_DONE = 3, TS_ADVANCE = 4, TS_ERROR = 5, TS_VALID = 6, TS_CAP = 7,
       TS_SYMS = 8, TS_MAXSYM = 9, TS_WORDS = 16 };

// Every decoder kernel serves a batch of utterances that step together: blockIdx.y is the utterance, its state words are
// state + b * TS_WORDS, its rows of the step buffers are `ld*` elements apart.

// xh0[b, 0:Hd] = table[state[b].token] when the prediction network of utterance b advances this step
__global__ void tdt_embed_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ state,
                                 __nv_bfloat16* __restrict__ xh0, int Hd, int rows, int ldx) {
  pdl_trigger();
  pdl_wait();
  const int* st = state + (size_t)blockIdx.y * TS_WORDS;
  if (st[TS_DONE] || !st[TS_ADVANCE]) return;
  const int tok = min(max(st[TS_TOKEN], 0), rows - 1);
  __nv_bfloat16* dst = xh0 + (size_t)blockIdx.y * ldx;
  for (int i = threadIdx.x; i < Hd; i += blockDim.x) dst[i] = table[(size_t)tok * Hd + i];
}

// gates: [batch, 4 Hd] BF16 pre-activations in i, f, g, o order (W [x; h]); bias: [4 Hd] FP32 (b_ih + b_hh).
// c: [batch, Hd] FP32 cell state. The new hidden state goes to h_self (the recurrent half of this layer's input) and
// h_next (the input half of the next layer, or the top output). Nothing is written when the step does not advance.
__global__ void lstm_cell_kernel(const __nv_bfloat16* __restrict__ gates, const float* __restrict__ bias,
                                 float* __restrict__ c, __nv_bfloat16* __restrict__ h_self,
                                 __nv_bfloat16* __restrict__ h_next, const int* __restrict__ state, int Hd, int ldg, int lds,
                                 int ldn) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.y;
  if (state != nullptr) {
    const int* st = state + (size_t)b * TS_WORDS;
    if (st[TS_DONE] || !st[TS_ADVANCE]) return;
  }
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= Hd) return;
  const __nv_bfloat16* g = gates + (size_t)b * ldg;
  float* cb = c + (size_t)b * Hd;
  const float gi = __bfloat162float(g[i]) + bias[i];
  const float gf = __bfloat162float(g[Hd + i]) + bias[Hd + i];
  const float gg = __bfloat162float(g[2 * Hd + i]) + bias[2 * Hd + i];
  const float go = __bfloat162float(g[3 * Hd + i]) + bias[3 * Hd + i];
  const float cn = sigmoidf_(gf) * cb[i] + sigmoidf_(gi) * tanhf(gg);
  const float hn = sigmoidf_(go) * tanhf(cn);
  cb[i] = cn;
  const __nv_bfloat16 hb = __float2bfloat16(hn);
  h_self[(size_t)b * lds + i] = hb;
  if (h_next) h_next[(size_t)b * ldn + i] = hb;
}

// out[b, j] = relu(enc[b, frame_b, j] + pred[b, j] + bias[j]) in BF16 (enc and pred are the two projections into the
// joint space; enc holds `frames` rows per utterance)
__global__ void tdt_joint_in_kernel(const __nv_bfloat16* __restrict__ enc, const __nv_bfloat16* __restrict__ pred,
                                    const float* __restrict__ bias, const int* __restrict__ state,
                                    __nv_bfloat16* __restrict__ out, int J, int frames, int ldp, int ldo) {
  pdl_trigger();
  pdl_wait();
  const int j = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (j >= J) return;
  const int f = min(max(state[(size_t)b * TS_WORDS + TS_FRAME], 0), frames - 1);
  const float x = __bfloat162float(enc[((size_t)b * frames + f) * J + j]) + __bfloat162float(pred[(size_t)b * ldp + j]) +
                  (bias ? bias[j] : 0.f);
  out[(size_t)b * ldo + j] = __float2bfloat16(fmaxf(x, 0.f));
}

// One greedy step per utterance: token = argmax logits[0 .. vocab] (index vocab is blank), duration = durations[argmax of
// the n_dur logits after it]; a blank with duration 0 moves one frame, and so does the TS_MAXSYM-th token in a row that
// would stay on its frame (the transducer's symbols-per-step limit). The trajectory entry and the next
// (frame, token) are written on the device. Lowest index wins ties. 256 threads, one CTA per utterance.
__global__ void __launch_bounds__(256)
tdt_select_kernel(const __nv_bfloat16* __restrict__ logits_all, const float* __restrict__ out_bias,
                  const int* __restrict__ durations, int* __restrict__ state_all, int* __restrict__ traj_tokens,
                  int* __restrict__ traj_durations, int* __restrict__ traj_frames, int n_tok, int n_dur, int blank, int eos,
                  int traj_len, int ldl) {
  pdl_trigger();
  pdl_wait();
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  const int ub = blockIdx.y;
  int* state = state_all + (size_t)ub * TS_WORDS;
  const __nv_bfloat16* logits = logits_all + (size_t)ub * ldl;
  traj_tokens += (size_t)ub * traj_len; traj_durations += (size_t)ub * traj_len; traj_frames += (size_t)ub * traj_len;
  if (state[TS_DONE]) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float best = -3.0e38f; int bi = 0x7fffffff;
  for (int i = tid; i < n_tok; i += 256) {
    const float x = __bfloat162float(logits[i]) + (out_bias ? out_bias[i] : 0.f);
    if (x > best) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = bi; }
  __syncthreads();
  if (tid != 0) return;
  for (int w = 1; w < 8; ++w)
    if (s_val[w] > best || (s_val[w] == best && s_idx[w] < bi)) { best = s_val[w]; bi = s_idx[w]; }
  float dbest = -3.0e38f; int di = 0;
  for (int i = 0; i < n_dur; ++i) {
    const float x = __bfloat162float(logits[n_tok + i]) + (out_bias ? out_bias[n_tok + i] : 0.f);
    if (x > dbest) { dbest = x; di = i; }
  }
  const int count = state[TS_COUNT], frame = state[TS_FRAME];
  // n_dur == 0: a plain transducer (no duration head): tokens stay on the frame, blanks move one frame
  const int valid_rows = state[TS_VALID], capacity = min(state[TS_CAP], traj_len);
  if (count >= capacity) { state[TS_ERROR] = 1; state[TS_DONE] = 1; return; }
  int dur = n_dur > 0 ? durations[di] : 0;
  if (bi == blank && dur == 0) dur = 1;
  int syms = state[TS_SYMS];
  if (bi != blank && dur == 0 && ++syms >= state[TS_MAXSYM]) dur = 1;
  state[TS_SYMS] = dur > 0 ? 0 : syms;
  traj_tokens[count] = bi; traj_durations[count] = dur; traj_frames[count] = frame;
  state[TS_COUNT] = count + 1;
  const int next = frame + dur;
  // the next (frame, token) is written even when the rows run out: a streaming decode resumes from it when more rows
  // arrive
  state[TS_FRAME] = next;
  state[TS_TOKEN] = bi;
  state[TS_ADVANCE] = bi != blank;
  if (bi == eos || next >= valid_rows) state[TS_DONE] = 1;
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_logmel(const float* wave, const int* lens, const float* window, const float* filters,
                        const int* band_range, float* out, int batch, long long max_samples, int frames, int n_fft,
                        int hop, int mel_bins, float preemph, float log_guard, cudaStream_t s) {
  if (batch <= 0 || frames <= 0 || n_fft < 32 || n_fft > MEL_MAX_FFT || (n_fft & (n_fft - 1)) || hop <= 0 || mel_bins <= 0)
    return FF_HOST_BAD_SHAPE;
  int log2n = 0;
  while ((1 << log2n) < n_fft) ++log2n;
  logmel_kernel<<<dim3(frames, batch), 256, 0, s>>>(wave, lens, window, filters, band_range, out, max_samples, frames,
                                                   n_fft, log2n, hop, mel_bins, preemph, log_guard);
  return launch_result();
}

FF_EXPORT int ff_feat_normalize(float* feat, const int* lens, int batch, int frames, int mel_bins, int hop, float eps,
                                cudaStream_t s) {
  if (batch <= 0 || frames <= 0 || mel_bins <= 0 || hop <= 0) return FF_HOST_BAD_SHAPE;
  feat_normalize_kernel<<<dim3((mel_bins + 31) / 32, batch), dim3(32, 8), 0, s>>>(feat, lens, frames, mel_bins, hop, eps);
  return launch_result();
}

FF_EXPORT int ff_sub_conv_first(const float* in, const float* w, const float* bias, const int* valid_out, void* out,
                                int batch, int T, int F, int T1, int F1, int C, int pad_t, int pad_f, cudaStream_t s) {
  if (batch <= 0 || T <= 0 || F <= 0 || T1 <= 0 || F1 <= 0 || C <= 0 || C % 8) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)batch * T1 * F1 * (C / 8);
  if (int lr = launch_pdl(sub_conv_first_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0, in, w, bias,
                          valid_out, (__nv_bfloat16*)out, T, F, T1, F1, C, pad_t, pad_f, total)) return lr;
  return launch_result();
}

FF_EXPORT int ff_sub_dwconv(const void* in, const float* w, const float* bias, const int* valid_in, void* out, int batch,
                            int T, int F, int T1, int F1, int C, int pad_t, int pad_f, cudaStream_t s) {
  if (batch <= 0 || T <= 0 || F <= 0 || T1 <= 0 || F1 <= 0 || C <= 0 || C % 8) return FF_HOST_BAD_SHAPE;
  const long long total = (long long)batch * T1 * F1 * (C / 8);
  if (int lr = launch_pdl(sub_dwconv_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)in, w, bias, valid_in, (__nv_bfloat16*)out, T, F, T1, F1, C, pad_t, pad_f,
                          total)) return lr;
  return launch_result();
}

FF_EXPORT int ff_glu_dwconv1d(const void* x, const float* xbias, const float* w, const float* bias, const int* lens,
                              void* y, int batch, int T, int H, int K, int left, int silu, cudaStream_t s) {
  if (batch <= 0 || T <= 0 || H <= 0 || H % 2 || K <= 0 || K > DW_MAX_K || left < 0 || left >= K) return FF_HOST_BAD_SHAPE;
  const dim3 grid((H / 2 + 127) / 128, (T + DW_STRIP - 1) / DW_STRIP, batch);
  int lr;
  if (K <= 9) lr = launch_pdl(glu_dwconv1d_kernel<9>, grid, dim3(128), 0, s, 0, (const __nv_bfloat16*)x, xbias, w, bias, lens,
                              (__nv_bfloat16*)y, T, H, K, left, silu);
  else lr = launch_pdl(glu_dwconv1d_kernel<DW_MAX_K>, grid, dim3(128), 0, s, 0, (const __nv_bfloat16*)x, xbias, w, bias, lens,
                       (__nv_bfloat16*)y, T, H, K, left, silu);
  if (lr) return lr;
  return launch_result();
}

FF_EXPORT int ff_scale_add_layernorm(void* h, const void* delta, const float* dbias, const float* w, const float* b,
                                     void* y, int rows, int hidden, int ldh, int ldd, int ldy, float scale, float eps,
                                     cudaStream_t s) {
  if (rows <= 0 || hidden <= 0 || hidden % 4 || hidden > 128 * 4 * SAL_MAX || ldh % 4 || ldd % 4 || ldy % 4)
    return FF_HOST_BAD_SHAPE;
  if (y != nullptr && w == nullptr) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(scale_add_layernorm_kernel, dim3(rows), dim3(128), 0, s, 0, (__nv_bfloat16*)h,
                          (const __nv_bfloat16*)delta, dbias, w, b, (__nv_bfloat16*)y, hidden, ldh, ldd, ldy, scale, eps))
    return lr;
  return launch_result();
}

FF_EXPORT int ff_relpos_attention(const void* q, const void* k, const void* v, const void* pos, const float* bias_u,
                                  const float* bias_v, const int* lens, void* out, int batch, int T, int heads,
                                  int head_dim, int ldq, int ldk, int ldv, int ldp, int ldo, int left, int right,
                                  int chunk, float scale, cudaStream_t s) {
  if (batch <= 0 || T <= 0 || heads <= 0 || (head_dim != 64 && head_dim != 128) || !(scale > 0.f)) return FF_HOST_BAD_SHAPE;
  if (chunk < 0 || (chunk > 0 && (left < 0 || right < 0))) return FF_HOST_BAD_SHAPE;
  if (ldq % 8 || ldk % 8 || ldv % 8 || ldp % 8 || ldo % 2) return FF_HOST_BAD_ALIGN;
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(k) & 15) || (reinterpret_cast<uintptr_t>(v) & 15) ||
      (reinterpret_cast<uintptr_t>(pos) & 15) || (reinterpret_cast<uintptr_t>(out) & 3)) return FF_HOST_BAD_ALIGN;
  const dim3 grid((T + RA_Q - 1) / RA_Q, heads, batch);
  const float sl2 = scale * 1.4426950408889634f;
  if (head_dim == 128) {
    constexpr int smem = ra_smem_bytes<128>();
    if (int e = opt_in_smem(relpos_attention_kernel<128>, smem)) return e;
    if (int lr = launch_pdl(relpos_attention_kernel<128>, grid, dim3(128), smem, s, 0, (const __nv_bfloat16*)q,
                            (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)pos, bias_u, bias_v,
                            lens, (__nv_bfloat16*)out, T, ldq, ldk, ldv, ldp, ldo, left, right, chunk, sl2)) return lr;
  } else {
    constexpr int smem = ra_smem_bytes<64>();
    if (int e = opt_in_smem(relpos_attention_kernel<64>, smem)) return e;
    if (int lr = launch_pdl(relpos_attention_kernel<64>, grid, dim3(128), smem, s, 0, (const __nv_bfloat16*)q,
                            (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)pos, bias_u, bias_v,
                            lens, (__nv_bfloat16*)out, T, ldq, ldk, ldv, ldp, ldo, left, right, chunk, sl2)) return lr;
  }
  return launch_result();
}

FF_EXPORT int ff_tdt_embed(const void* table, const int* state, void* xh0, int batch, int Hd, int rows, int ldx,
                           cudaStream_t s) {
  if (batch <= 0 || Hd <= 0 || rows <= 0 || ldx < Hd) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(tdt_embed_kernel, dim3(1, batch), dim3(256), 0, s, 0, (const __nv_bfloat16*)table, state,
                          (__nv_bfloat16*)xh0, Hd, rows, ldx)) return lr;
  return launch_result();
}

FF_EXPORT int ff_lstm_cell(const void* gates, const float* bias, float* c, void* h_self, void* h_next, const int* state,
                           int batch, int Hd, int ldg, int lds, int ldn, cudaStream_t s) {
  if (batch <= 0 || Hd <= 0 || ldg < 4 * Hd || lds < Hd) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(lstm_cell_kernel, dim3((Hd + 127) / 128, batch), dim3(128), 0, s, 0, (const __nv_bfloat16*)gates,
                          bias, c, (__nv_bfloat16*)h_self, (__nv_bfloat16*)h_next, state, Hd, ldg, lds, ldn)) return lr;
  return launch_result();
}

FF_EXPORT int ff_tdt_joint_in(const void* enc, const void* pred, const float* bias, const int* state, void* out, int batch,
                              int J, int frames, int ldp, int ldo, cudaStream_t s) {
  if (batch <= 0 || J <= 0 || frames <= 0 || ldp < J || ldo < J) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(tdt_joint_in_kernel, dim3((J + 127) / 128, batch), dim3(128), 0, s, 0, (const __nv_bfloat16*)enc,
                          (const __nv_bfloat16*)pred, bias, state, (__nv_bfloat16*)out, J, frames, ldp, ldo)) return lr;
  return launch_result();
}

FF_EXPORT int ff_tdt_select(const void* logits, const float* out_bias, const int* durations, int* state, int* traj_tokens,
                            int* traj_durations, int* traj_frames, int batch, int n_tok, int n_dur, int blank, int eos,
                            int traj_len, int ldl, cudaStream_t s) {
  if (batch <= 0 || n_tok <= 0 || n_dur < 0 || traj_len <= 0 || ldl < n_tok + n_dur) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(tdt_select_kernel, dim3(1, batch), dim3(256), 0, s, 0, (const __nv_bfloat16*)logits, out_bias,
                          durations, state, traj_tokens, traj_durations, traj_frames, n_tok, n_dur, blank, eos, traj_len, ldl))
    return lr;
  return launch_result();
}
