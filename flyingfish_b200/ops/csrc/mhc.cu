// Manifold-constrained hyper-connections (mHC): the residual is `mult` parallel streams per token.
// Around every sub-layer:
//   mixes   : r = rsqrt(mean(x^2) + norm_eps) over all mult*hidden elements of the row;
//             mix[c] = (fn[c] . x) * r for the (2 + mult) * mult mixer rows;
//             pre[j]  = sigmoid(mix[j] * scale0 + base[j]) + eps
//             post[j] = 2 * sigmoid(mix[mult + j] * scale1 + base[mult + j])
//             comb    = Sinkhorn(softmax_rows(mix[2 mult ..] * scale2 + base[2 mult ..]) + eps): one column
//                       normalisation, then (iters - 1) row + column normalisations, every divide by (sum + eps)
//   collapse: y[h] = sum_j pre[j] * x[j, h]                       (the sub-layer's input)
//   update  : x'[j, h] = post[j] * f[h] + sum_k coeff(j, k) * x[k, h] with coeff = comb (orientation 0)
//             or comb transposed (orientation 1); rounding 0 = FP32 products and adds, one BF16 round;
//             rounding 1 = BF16 post, BF16 product, BF16-rounded coefficients with FP32 accumulation and
//             a BF16 round, BF16 add.
// Restates kernels/mhc.cu of the reference (:1-37 contract, :60-125 finish, :127-170 mixes,
// :300-438 collapse / update). Here the mixer dot products of a row are computed by one CTA with the
// row staged in shared memory and each warp owning mixer rows (no block-wide reduction per mixer row).
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int MHC_MAX_MULT = 8;

// grid rows, 256 threads; dynamic smem = mult*hidden bf16
__global__ void __launch_bounds__(256)
mhc_mixes_kernel(const __nv_bfloat16* __restrict__ stream, const __nv_bfloat16* __restrict__ fn,
                 const float* __restrict__ base, const float* __restrict__ scale, int mult, int hidden, int iters,
                 float eps, float norm_eps, float* __restrict__ pre, float* __restrict__ post, float* __restrict__ comb) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(16) uint8_t mhc_smem[];
  __nv_bfloat16* sx = reinterpret_cast<__nv_bfloat16*>(mhc_smem);
  __shared__ float s_red[8];
  __shared__ float s_mix[(2 + MHC_MAX_MULT) * MHC_MAX_MULT];
  __shared__ float s_comb[MHC_MAX_MULT * MHC_MAX_MULT];
  const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = mult * hidden, nmix = (2 + mult) * mult;
  const uint4* src = reinterpret_cast<const uint4*>(stream + (size_t)row * n);
  float sumsq = 0.f;
  for (int i = tid; i < n / 8; i += 256) {
    const uint4 v = src[i];
    reinterpret_cast<uint4*>(sx)[i] = v;
    const uint32_t* p = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(p[j]); sumsq += f.x * f.x + f.y * f.y; }
  }
  sumsq = warp_sum(sumsq);
  if (lane == 0) s_red[warp] = sumsq;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += s_red[w];
  const float r = 1.0f / sqrtf(tot / (float)n + norm_eps);
  for (int c = warp; c < nmix; c += 8) {
    const uint4* frow = reinterpret_cast<const uint4*>(fn + (size_t)c * n);
    float acc = 0.f;
    for (int i = lane; i < n / 8; i += 32) {
      const uint4 fv = frow[i], xv = reinterpret_cast<const uint4*>(sx)[i];
      const uint32_t* fp = reinterpret_cast<const uint32_t*>(&fv); const uint32_t* xp = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 a = unpack_bf16x2(fp[j]), b = unpack_bf16x2(xp[j]); acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); }
    }
    acc = warp_sum(acc);
    if (lane == 0) s_mix[c] = acc * r;
  }
  __syncthreads();
  if (tid == 0) {
    for (int j = 0; j < mult; ++j) {
      pre[(size_t)row * mult + j] = 1.0f / (1.0f + expf(-(s_mix[j] * scale[0] + base[j]))) + eps;
      post[(size_t)row * mult + j] = 2.0f * (1.0f / (1.0f + expf(-(s_mix[mult + j] * scale[1] + base[mult + j]))));
    }
    for (int j = 0; j < mult; ++j) {
      float mx = -INFINITY;
      for (int k = 0; k < mult; ++k) { s_comb[j * mult + k] = s_mix[2 * mult + j * mult + k] * scale[2] + base[2 * mult + j * mult + k]; mx = fmaxf(mx, s_comb[j * mult + k]); }
      float rowsum = 0.f;
      for (int k = 0; k < mult; ++k) { const float e = expf(s_comb[j * mult + k] - mx); s_comb[j * mult + k] = e; rowsum += e; }
      for (int k = 0; k < mult; ++k) s_comb[j * mult + k] = s_comb[j * mult + k] / rowsum + eps;
    }
    for (int it = 0; it < iters; ++it) {
      if (it > 0)
        for (int j = 0; j < mult; ++j) {
          float rowsum = 0.f;
          for (int k = 0; k < mult; ++k) rowsum += s_comb[j * mult + k];
          for (int k = 0; k < mult; ++k) s_comb[j * mult + k] = s_comb[j * mult + k] / (rowsum + eps);
        }
      for (int k = 0; k < mult; ++k) {
        float colsum = 0.f;
        for (int j = 0; j < mult; ++j) colsum += s_comb[j * mult + k];
        for (int j = 0; j < mult; ++j) s_comb[j * mult + k] = s_comb[j * mult + k] / (colsum + eps);
      }
    }
    for (int i = 0; i < mult * mult; ++i) comb[(size_t)row * mult * mult + i] = s_comb[i];
  }
}

__global__ void mhc_collapse_kernel(const __nv_bfloat16* __restrict__ stream, const float* __restrict__ pre, int mult,
                                    int hidden, __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= hidden) return;
  float acc = 0.f;
  for (int j = 0; j < mult; ++j)
    acc = __fadd_rn(acc, __fmul_rn(pre[(size_t)row * mult + j], __bfloat162float(stream[((size_t)row * mult + j) * hidden + h])));
  out[(size_t)row * hidden + h] = __float2bfloat16_rn(acc);
}

__global__ void mhc_update_kernel(const __nv_bfloat16* __restrict__ sub, const __nv_bfloat16* __restrict__ residual,
                                  const float* __restrict__ post, const float* __restrict__ comb, int mult, int hidden,
                                  int rounding, int orientation, __nv_bfloat16* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.y, h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= hidden) return;
  const float f = __bfloat162float(sub[(size_t)row * hidden + h]);
  float res[MHC_MAX_MULT];
  for (int k = 0; k < mult; ++k) res[k] = __bfloat162float(residual[((size_t)row * mult + k) * hidden + h]);
  for (int j = 0; j < mult; ++j) {
    float o;
    if (rounding == 1) {
      const float p = __bfloat162float(__float2bfloat16_rn(post[(size_t)row * mult + j]));
      const float prod = __bfloat162float(__float2bfloat16_rn(p * f));
      float acc = 0.f;
      for (int k = 0; k < mult; ++k) {
        const float c = __bfloat162float(__float2bfloat16_rn(comb[(size_t)row * mult * mult + (orientation == 0 ? j * mult + k : k * mult + j)]));
        acc = fmaf(c, res[k], acc);
      }
      o = prod + __bfloat162float(__float2bfloat16_rn(acc));
    } else {
      o = __fmul_rn(post[(size_t)row * mult + j], f);
      for (int k = 0; k < mult; ++k)
        o = __fadd_rn(o, __fmul_rn(comb[(size_t)row * mult * mult + (orientation == 0 ? j * mult + k : k * mult + j)], res[k]));
    }
    out[((size_t)row * mult + j) * hidden + h] = __float2bfloat16_rn(o);
  }
}

}  // namespace ff
using namespace ff;

// stream [rows, mult, hidden] bf16; fn [(2+mult)*mult, mult*hidden] bf16; base [(2+mult)*mult] f32; scale [3] f32
FF_EXPORT int ff_mhc_mixes(const void* stream, const void* fn, const float* base, const float* scale, int rows, int mult,
                           int hidden, int iters, float eps, float norm_eps, float* pre, float* post, float* comb,
                           cudaStream_t s) {
  if (rows <= 0 || mult < 2 || mult > MHC_MAX_MULT || hidden <= 0 || hidden % 8 || iters < 1 || !(eps > 0.f) || !(norm_eps > 0.f))
    return FF_HOST_BAD_SHAPE;
  const int smem = mult * hidden * 2;
  if (smem > 200 * 1024) return FF_HOST_TOO_LARGE;
  if (int r = opt_in_smem(mhc_mixes_kernel, smem)) return r;
  if (int lr = launch_pdl(mhc_mixes_kernel, dim3(rows), dim3(256), smem, s, 0, (const __nv_bfloat16*)stream, (const __nv_bfloat16*)fn,
                          base, scale, mult, hidden, iters, eps, norm_eps, pre, post, comb)) return lr;
  return launch_result();
}

FF_EXPORT int ff_mhc_collapse(const void* stream, const float* pre, int rows, int mult, int hidden, void* out, cudaStream_t s) {
  if (rows <= 0 || mult < 2 || mult > MHC_MAX_MULT || hidden <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(mhc_collapse_kernel, dim3((hidden + 255) / 256, rows), dim3(256), 0, s, 0, (const __nv_bfloat16*)stream, pre,
                          mult, hidden, (__nv_bfloat16*)out)) return lr;
  return launch_result();
}

FF_EXPORT int ff_mhc_update(const void* sub, const void* residual, const float* post, const float* comb, int rows, int mult,
                            int hidden, int rounding, int orientation, void* out, cudaStream_t s) {
  if (rows <= 0 || mult < 2 || mult > MHC_MAX_MULT || hidden <= 0 || (unsigned)rounding > 1u || (unsigned)orientation > 1u)
    return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(mhc_update_kernel, dim3((hidden + 255) / 256, rows), dim3(256), 0, s, 0, (const __nv_bfloat16*)sub,
                          (const __nv_bfloat16*)residual, post, comb, mult, hidden, rounding, orientation, (__nv_bfloat16*)out)) return lr;
  return launch_result();
}
