// Row-wise normalisation family, all memory-bound: BF16 I/O, FP32 math, 16-byte vectors,
// one pass with the row cached in registers.
//   embed_rmsnorm      : x[r] = table[ids[r]] ; n[r] = rmsnorm(x[r]) * w
//   rmsnorm            : n[r] = rmsnorm(x[r]) * w
//   add_rmsnorm        : res[r] = bf16(res[r] + x[r]) ; n[r] = rmsnorm(res[r]) * w
//                        (the ROUNDED sum is what gets normalised; the product x*rstd*w is
//                        rounded once) with an optional copy of the new residual into a capture
//                        slab [rows, taps, hidden] for a draft model.
// Numerics follow the reference's contract (kernels/norm.cu:8-21, kernels/embed_rmsnorm.cu:1-22,
// kernels/add_rmsnorm_capture.cu).
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 8;   // 256 threads * 8 vectors * 8 bf16 = hidden up to 16384

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (blockDim.x >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// mode: 0 = rmsnorm(x), 1 = embed gather then norm, 2 = add + norm
// unit_offset: 1 -> weight is (1 + w) (Gemma convention), 0 -> w
template <int MODE>
__global__ void __launch_bounds__(NORM_THREADS)
norm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ res, const int* __restrict__ ids,
            const __nv_bfloat16* __restrict__ table, const __nv_bfloat16* __restrict__ w,
            __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ capture, int capture_stride, int hidden,
            int vocab, float eps, int unit_offset, int ldx, int* status) {
  pdl_trigger();
  if (threadIdx.x == 0) FF_TL(status, KID_NORM, 0);
  pdl_wait();
  if (threadIdx.x == 0) FF_TL(status, KID_NORM, 1);
  __shared__ float red[32];
  const int row = blockIdx.x;
  const int nvec = hidden >> 3;
  const __nv_bfloat16* src;
  if (MODE == 1) {
    int id = ids[row];
    if (id < 0 || id >= vocab) { set_status(status, KID_EMBED, FF_ERR_BOUNDS, row, id); id = 0; }
    src = table + (size_t)id * hidden;
  } else {
    src = x + (size_t)row * ldx;
  }
  uint4 v[NORM_MAX_VEC];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * NORM_THREADS;
    if (idx < nvec) {
      uint4 a = reinterpret_cast<const uint4*>(src)[idx];
      if (MODE == 2) {
        uint4 r = reinterpret_cast<const uint4*>(res + (size_t)row * hidden)[idx];
        uint32_t* ap = reinterpret_cast<uint32_t*>(&a);
        const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 fa = unpack_bf16x2(ap[j]), fr = unpack_bf16x2(rp[j]);
          ap[j] = pack_bf16x2(fa.x + fr.x, fa.y + fr.y);   // residual rounded to BF16 first
        }
        reinterpret_cast<uint4*>(res + (size_t)row * hidden)[idx] = a;
        if (capture) reinterpret_cast<uint4*>(capture + (size_t)row * capture_stride)[idx] = a;
      } else if (MODE == 1) {
        reinterpret_cast<uint4*>(res + (size_t)row * hidden)[idx] = a;
      }
      v[i] = a;
      const uint32_t* ap = reinterpret_cast<const uint32_t*>(&a);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(ap[j]); ss += f.x * f.x + f.y * f.y; }
    }
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)hidden + eps);
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i) {
    const int idx = threadIdx.x + i * NORM_THREADS;
    if (idx < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(w)[idx];
      const uint32_t* ap = reinterpret_cast<const uint32_t*>(&v[i]);
      const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
      uint4 o; uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf16x2(ap[j]), g = unpack_bf16x2(wp[j]);
        if (unit_offset) { g.x += 1.f; g.y += 1.f; }
        op[j] = pack_bf16x2(f.x * rstd * g.x, f.y * rstd * g.y);
      }
      reinterpret_cast<uint4*>(out + (size_t)row * hidden)[idx] = o;
    }
  }
}

// plain residual add: res = bf16(res + x)
__global__ void residual_add_kernel(__nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ x, size_t nvec) {
  pdl_trigger();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nvec) return;
  uint4 a = reinterpret_cast<const uint4*>(x)[i], r = reinterpret_cast<uint4*>(res)[i];
  uint32_t* ap = reinterpret_cast<uint32_t*>(&a); const uint32_t* rp = reinterpret_cast<const uint32_t*>(&r);
#pragma unroll
  for (int j = 0; j < 4; ++j) { float2 fa = unpack_bf16x2(ap[j]), fr = unpack_bf16x2(rp[j]); ap[j] = pack_bf16x2(fa.x + fr.x, fa.y + fr.y); }
  reinterpret_cast<uint4*>(res)[i] = a;
}

// plain embedding gather (no norm): out[r] = table[ids[r]] * scale
__global__ void embed_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                             __nv_bfloat16* __restrict__ out, int hidden, int vocab, float scale, int* status) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) { set_status(status, KID_EMBED, FF_ERR_BOUNDS, row, id); id = 0; }
  const int nvec = hidden >> 3;
  for (int idx = threadIdx.x; idx < nvec; idx += blockDim.x) {
    uint4 a = reinterpret_cast<const uint4*>(table + (size_t)id * hidden)[idx];
    if (scale != 1.0f) {
      uint32_t* ap = reinterpret_cast<uint32_t*>(&a);
#pragma unroll
      for (int j = 0; j < 4; ++j) { float2 f = unpack_bf16x2(ap[j]); ap[j] = pack_bf16x2(f.x * scale, f.y * scale); }
    }
    reinterpret_cast<uint4*>(out + (size_t)row * hidden)[idx] = a;
  }
}

}  // namespace ff
using namespace ff;

static int check_hidden(int hidden) {
  if (hidden <= 0 || (hidden % 8) || hidden > NORM_THREADS * NORM_MAX_VEC * 8) return FF_HOST_BAD_SHAPE;
  return 0;
}

FF_EXPORT int ff_rmsnorm(const void* x, const void* w, void* out, int rows, int hidden, int ldx, float eps,
                         int unit_offset, int* status, cudaStream_t s) {
  if (int r = check_hidden(hidden)) return r;
  if (rows <= 0) return FF_HOST_BAD_SHAPE;
  if (ldx % 8) return FF_HOST_BAD_ALIGN;
  if (int lr_ = launch_pdl(norm_kernel<0>, dim3(rows), dim3(NORM_THREADS), 0, s, 0, (const __nv_bfloat16*)x, nullptr, nullptr, nullptr,
      (const __nv_bfloat16*)w, (__nv_bfloat16*)out, nullptr, 0, hidden, 0, eps, unit_offset, ldx, status)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_embed_rmsnorm(const int* ids, const void* table, const void* w, void* res, void* out, int rows,
                               int hidden, int vocab, float eps, int unit_offset, int* status, cudaStream_t s) {
  if (int r = check_hidden(hidden)) return r;
  if (rows <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr_ = launch_pdl(norm_kernel<1>, dim3(rows), dim3(NORM_THREADS), 0, s, 0, nullptr, (__nv_bfloat16*)res, ids, (const __nv_bfloat16*)table,
      (const __nv_bfloat16*)w, (__nv_bfloat16*)out, nullptr, 0, hidden, vocab, eps, unit_offset, hidden, status)) return lr_;
  return launch_result();
}

// capture may be null; capture_stride is the element stride between rows of the capture slab
// (taps * hidden) with the tap offset already applied to the pointer.
FF_EXPORT int ff_add_rmsnorm(const void* x, void* res, const void* w, void* out, void* capture, int capture_stride,
                             int rows, int hidden, int ldx, float eps, int unit_offset, int* status, cudaStream_t s) {
  if (int r = check_hidden(hidden)) return r;
  if (rows <= 0) return FF_HOST_BAD_SHAPE;
  if (ldx % 8 || capture_stride % 8) return FF_HOST_BAD_ALIGN;
  if (int lr_ = launch_pdl(norm_kernel<2>, dim3(rows), dim3(NORM_THREADS), 0, s, 0, (const __nv_bfloat16*)x, (__nv_bfloat16*)res, nullptr, nullptr,
      (const __nv_bfloat16*)w, (__nv_bfloat16*)out, (__nv_bfloat16*)capture, capture_stride, hidden, 0, eps,
      unit_offset, ldx, status)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_residual_add(void* res, const void* x, long long n, cudaStream_t s) {
  if (n <= 0 || (n % 8)) return FF_HOST_BAD_SHAPE;
  const size_t nvec = (size_t)n / 8;
  if (int lr_ = launch_pdl(residual_add_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, s, 0, (__nv_bfloat16*)res, (const __nv_bfloat16*)x, nvec)) return lr_;
  return launch_result();
}

FF_EXPORT int ff_embed(const int* ids, const void* table, void* out, int rows, int hidden, int vocab, float scale,
                       int* status, cudaStream_t s) {
  if (rows <= 0 || hidden <= 0 || (hidden % 8)) return FF_HOST_BAD_SHAPE;
  if (int lr_ = launch_pdl(embed_kernel, dim3(rows), dim3(256), 0, s, 0, ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, hidden, vocab, scale, status)) return lr_;
  return launch_result();
}
