// Quantisation kernels (memory-bound, one pass):
//   quant_fp8_1x128   : BF16 activations -> E4M3 codes + one FP32 scale per 128 elements
//                       (scale = amax / 448, zero groups get scale 1), the activation side of the
//                       block-scaled FP8 linear (kernels/fp8_linear.cu:12-48 of the reference);
//                       `ue8m0` != 0 switches to the DeepSeek form: amax floored at 1e-4 and the
//                       scale rounded up to a power of two (kernels/q38_contract.cuh:153-170)
//   dequant_fp8_block : E4M3 codes with 128x128 block scales -> BF16
//   dequant_nvfp4     : packed E2M1 + E4M3 scale per 16 + FP32 global scale -> BF16 effective
//                       weights (kernels/nvfp4_linear.cu `nvfp4_dequant_bf16`, src/fp8.rs:124-147)
//   quant_nvfp4 / quant_mxfp4 : BF16 -> packed E2M1 with E4M3-per-16 or E8M0-per-32 scales
//                       (kernels/quantize.cu fp4_pack_e4m3_16 / fp4_pack_e8m0_32)
#include "ptx.cuh"
#include "host_util.h"
#include <cuda_fp8.h>

namespace ff {

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(uint8_t c) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}
__device__ __forceinline__ float e2m1_value(uint32_t code) {
  const float mags[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float m = mags[code & 7];
  return (code & 8) ? -m : m;
}
// nearest E2M1 magnitude index, ties to the even index
__device__ __forceinline__ uint32_t e2m1_code(float v) {
  const float a = fminf(fabsf(v), 6.0f);
  uint32_t idx;
  if (a <= 0.25f) idx = 0; else if (a < 0.75f) idx = 1; else if (a <= 1.25f) idx = 2; else if (a < 1.75f) idx = 3;
  else if (a <= 2.5f) idx = 4; else if (a < 3.5f) idx = 5; else if (a <= 5.0f) idx = 6; else idx = 7;
  return idx | (v < 0.f ? 8u : 0u);
}

// one warp per (row, 128-group): lane holds 4 consecutive elements
__global__ void quant_fp8_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                       float* __restrict__ scale, int rows, int K, int ldx, int ue8m0, long long ldq,
                                       long long lds) {
  pdl_trigger();
  pdl_wait();
  const int groups = K >> 7;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)rows * groups) return;
  const int row = (int)(wid / groups), g = (int)(wid % groups);
  const uint2 raw = *reinterpret_cast<const uint2*>(x + (size_t)row * ldx + g * 128 + lane * 4);
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_max(amax);
  float s;
  if (ue8m0) { amax = fmaxf(amax, 1e-4f); s = exp2f(ceilf(log2f(amax / 448.0f))); }
  else s = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  // true division (not a reciprocal multiply) so the codes match the host codec bit for bit
  const uint32_t packed = (uint32_t)to_e4m3(__fdiv_rn(a.x, s)) | ((uint32_t)to_e4m3(__fdiv_rn(a.y, s)) << 8) |
                          ((uint32_t)to_e4m3(__fdiv_rn(b.x, s)) << 16) | ((uint32_t)to_e4m3(__fdiv_rn(b.y, s)) << 24);
  *reinterpret_cast<uint32_t*>(q + (size_t)row * ldq + g * 128 + lane * 4) = packed;
  if (lane == 0) scale[(size_t)row * lds + g] = s;
}

__global__ void dequant_fp8_block_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                                         __nv_bfloat16* __restrict__ out, int N, int K, int scale_cols) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= (long long)N * K) return;
  const int n = (int)(i / K), k = (int)(i % K);
  const float s = scale[(size_t)(n >> 7) * scale_cols + (k >> 7)];
  const uint32_t c = *reinterpret_cast<const uint32_t*>(q + i);
  uint2 o;
  o.x = pack_bf16x2(from_e4m3(c & 0xff) * s, from_e4m3((c >> 8) & 0xff) * s);
  o.y = pack_bf16x2(from_e4m3((c >> 16) & 0xff) * s, from_e4m3(c >> 24) * s);
  *reinterpret_cast<uint2*>(out + i) = o;
}

// one thread per group of 16 weights (8 packed bytes)
__global__ void dequant_nvfp4_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                     const float* __restrict__ global_scale, __nv_bfloat16* __restrict__ out,
                                     long long groups) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const float s = from_e4m3(scales[g]) * global_scale[0];
  const uint2 p = *reinterpret_cast<const uint2*>(packed + g * 8);
  uint32_t o[8];
  const uint32_t w[2] = {p.x, p.y};
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (w[h] >> (8 * b)) & 0xff;
      o[h * 4 + b] = pack_bf16x2(e2m1_value(byte & 0xf) * s, e2m1_value(byte >> 4) * s);
    }
  uint4* dst = reinterpret_cast<uint4*>(out + g * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// BF16 -> packed E2M1. mode 0: NVFP4 (group 16, E4M3 scale relative to *global_scale),
// mode 1: MXFP4 (group 32, E8M0 scale, power of two >= amax/6). One thread per group.
__global__ void quant_fp4_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ packed,
                                 uint8_t* __restrict__ scales, const float* __restrict__ global_scale, long long groups,
                                 int mode) {
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= groups) return;
  const int gs = mode == 0 ? 16 : 32;
  const __nv_bfloat16* src = x + g * gs;
  float v[32];
  float amax = 0.f;
  for (int i = 0; i < gs; ++i) { v[i] = __bfloat162float(src[i]); amax = fmaxf(amax, fabsf(v[i])); }
  float s; uint8_t code;
  if (mode == 0) {
    const float gsv = global_scale[0];
    code = to_e4m3(amax / 6.0f / gsv);
    s = from_e4m3(code) * gsv;
  } else {
    const float e = ceilf(log2f(fmaxf(amax / 6.0f, 1.17549435e-38f)));
    const float ec = fminf(fmaxf(e + 127.f, 0.f), 254.f);
    code = (uint8_t)ec;
    s = exp2f(ec - 127.f);
  }
  if (!(s > 0.f)) s = 1.f;
  scales[g] = code;
  const float inv = 1.0f / s;
  for (int i = 0; i < gs; i += 2)
    packed[(g * gs + i) >> 1] = (uint8_t)(e2m1_code(v[i] * inv) | (e2m1_code(v[i + 1] * inv) << 4));
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_quant_fp8_1x128(const void* x, void* q, float* scale, int rows, int K, int ldx, int ue8m0,
                                 cudaStream_t s) {
  if (rows <= 0 || K <= 0 || K % 128 || ldx % 4) return FF_HOST_BAD_SHAPE;
  const long long warps = (long long)rows * (K / 128);
  if (int lr = launch_pdl(quant_fp8_1x128_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)x, (uint8_t*)q, scale, rows, K, ldx, ue8m0, (long long)K,
                          (long long)(K / 128))) return lr;
  return launch_result();
}

// The same quantisation into strided outputs: code rows ldq bytes apart, scale rows lds floats apart. With
// scale = (float*)(q + K), ldq = K + K / 32 and lds = ldq / 4 a row is one packed record [K codes | K / 128 scales]:
// the form in which token rows travel to the ranks that own their experts.
FF_EXPORT int ff_quant_fp8_1x128_strided(const void* x, void* q, float* scale, int rows, int K, int ldx, long long ldq,
                                         long long lds, cudaStream_t s) {
  if (rows <= 0 || K <= 0 || K % 128 || ldx % 4 || ldq < K || ldq % 4 || lds < K / 128) return FF_HOST_BAD_SHAPE;
  const long long warps = (long long)rows * (K / 128);
  if (int lr = launch_pdl(quant_fp8_1x128_kernel, dim3((unsigned)((warps * 32 + 255) / 256)), dim3(256), 0, s, 0,
                          (const __nv_bfloat16*)x, (uint8_t*)q, scale, rows, K, ldx, 0, ldq, lds)) return lr;
  return launch_result();
}

FF_EXPORT int ff_dequant_fp8_block(const void* q, const float* scale, void* out, int N, int K, cudaStream_t s) {
  if (N <= 0 || K <= 0 || K % 4) return FF_HOST_BAD_SHAPE;
  const long long n4 = (long long)N * K / 4;
  dequant_fp8_block_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, s>>>((const uint8_t*)q, scale, (__nv_bfloat16*)out, N, K,
                                                                         (K + 127) / 128);
  return launch_result();
}

FF_EXPORT int ff_dequant_nvfp4(const void* packed, const void* scales, const float* global_scale, void* out,
                               long long n_elems, cudaStream_t s) {
  if (n_elems <= 0 || n_elems % 16) return FF_HOST_BAD_SHAPE;
  const long long groups = n_elems / 16;
  dequant_nvfp4_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>((const uint8_t*)packed, (const uint8_t*)scales,
                                                                        global_scale, (__nv_bfloat16*)out, groups);
  return launch_result();
}

FF_EXPORT int ff_quant_fp4(const void* x, void* packed, void* scales, const float* global_scale, long long n_elems,
                           int mode, cudaStream_t s) {
  const int gs = mode == 0 ? 16 : 32;
  if (n_elems <= 0 || n_elems % gs || (mode == 0 && !global_scale)) return FF_HOST_BAD_SHAPE;
  const long long groups = n_elems / gs;
  quant_fp4_kernel<<<(unsigned)((groups + 127) / 128), 128, 0, s>>>((const __nv_bfloat16*)x, (uint8_t*)packed,
                                                                    (uint8_t*)scales, global_scale, groups, mode);
  return launch_result();
}
