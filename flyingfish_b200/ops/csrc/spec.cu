// Speculative-decoding helpers on the device.
//   mtp_mix      : input rows of a multi-token-prediction module: out[r] = [ rmsnorm(embed[ids[r]]) * enorm |
//                  rmsnorm(hidden[r]) * hnorm ]  (one launch instead of gather + two norms + concatenation; the
//                  concatenated row feeds the eh_proj GEMM). Same rounding as the stand-alone norm kernel: FP32 math,
//                  one BF16 rounding of x * rstd * w.
//   accept_chain : greedy acceptance of k draft tokens per sequence against the target's k+1 greedy tokens: the longest
//                  matching prefix plus the target's token at the first mismatch; an end-of-sequence token inside the
//                  accepted prefix ends the emission. out[b] = {accepted drafts, emitted count, hit_eos, tokens...}.
// Reference: the MTP module input and the batched acceptance of src/mtp/batched.rs:71-194, src/dspark.rs:932-950.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int MIX_THREADS = 256;
constexpr int MIX_MAX_VEC = 8;       // hidden <= 256 * 8 * 8

__device__ __forceinline__ float mix_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (MIX_THREADS >> 5)) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(MIX_THREADS)
mtp_mix_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, const __nv_bfloat16* __restrict__ hidden,
               const __nv_bfloat16* __restrict__ enorm, const __nv_bfloat16* __restrict__ hnorm,
               __nv_bfloat16* __restrict__ out, int hdim, int vocab, int ldh, float eps, int* status) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int row = blockIdx.x;
  int id = ids[row];
  if (id < 0 || id >= vocab) { if (threadIdx.x == 0) set_status(status, KID_EMBED, FF_ERR_BOUNDS, row, id); id = 0; }
  const int nvec = hdim >> 3;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const __nv_bfloat16* src = half == 0 ? table + (size_t)id * hdim : hidden + (size_t)row * ldh;
    const __nv_bfloat16* w = half == 0 ? enorm : hnorm;
    uint4 v[MIX_MAX_VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MIX_MAX_VEC; ++i) {
      const int idx = threadIdx.x + i * MIX_THREADS;
      if (idx < nvec) {
        v[i] = reinterpret_cast<const uint4*>(src)[idx];
        const uint32_t* ap = reinterpret_cast<const uint32_t*>(&v[i]);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(ap[j]); ss += f.x * f.x + f.y * f.y; }
      }
    }
    const float rstd = rsqrtf(mix_block_sum(ss, red) / (float)hdim + eps);
#pragma unroll
    for (int i = 0; i < MIX_MAX_VEC; ++i) {
      const int idx = threadIdx.x + i * MIX_THREADS;
      if (idx < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(w)[idx];
        const uint32_t* ap = reinterpret_cast<const uint32_t*>(&v[i]);
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(&wv);
        uint4 o; uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = unpack_bf16x2(ap[j]), g = unpack_bf16x2(wp[j]);
          op[j] = pack_bf16x2(f.x * rstd * g.x, f.y * rstd * g.y);
        }
        reinterpret_cast<uint4*>(out + (size_t)row * 2 * hdim + (size_t)half * hdim)[idx] = o;
      }
    }
  }
}

// one thread per sequence; out row: [n_accepted, n_emitted, hit_eos, tok_0 .. tok_k] (unused tokens -1)
__global__ void accept_chain_kernel(const int* __restrict__ draft, const int* __restrict__ target, const int* __restrict__ eos,
                                    int n_eos, int ignore_eos, int batch, int k, int* __restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const int* d = draft + (size_t)b * k;
  const int* t = target + (size_t)b * (k + 1);
  int* o = out + (size_t)b * (k + 4);
  auto is_eos = [&](int tok) { for (int i = 0; i < n_eos; ++i) if (eos[i] == tok) return true; return false; };
  int n = 0, emitted = 0, hit = 0;
  for (int j = 0; j <= k; ++j) o[3 + j] = -1;
  bool done = false;
  for (int j = 0; j < k && !done; ++j) {
    if (d[j] != t[j]) break;
    o[3 + emitted++] = d[j];
    ++n;
    if (!ignore_eos && is_eos(d[j])) { hit = 1; done = true; }
  }
  if (!done) {
    o[3 + emitted++] = t[n];
    if (!ignore_eos && is_eos(t[n])) hit = 1;
  }
  o[0] = n; o[1] = emitted; o[2] = hit;
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_mtp_mix(const int* ids, const void* table, const void* hidden, const void* enorm, const void* hnorm,
                         void* out, int rows, int hdim, int vocab, int ldh, float eps, int* status, cudaStream_t s) {
  if (rows <= 0 || hdim <= 0 || hdim % 8 || hdim > MIX_THREADS * 8 * MIX_MAX_VEC || ldh % 8) return FF_HOST_BAD_SHAPE;
  return launch_pdl(mtp_mix_kernel, dim3(rows), dim3(MIX_THREADS), 0, s, 0, ids, (const __nv_bfloat16*)table,
                    (const __nv_bfloat16*)hidden, (const __nv_bfloat16*)enorm, (const __nv_bfloat16*)hnorm,
                    (__nv_bfloat16*)out, hdim, vocab, ldh, eps, status);
}

// out: int32 [batch, k + 4]
FF_EXPORT int ff_accept_chain(const int* draft, const int* target, const int* eos, int n_eos, int ignore_eos, int batch,
                              int k, int* out, cudaStream_t s) {
  if (batch <= 0 || k < 0 || n_eos < 0) return FF_HOST_BAD_SHAPE;
  return launch_pdl(accept_chain_kernel, dim3((batch + 63) / 64), dim3(64), 0, s, 0, draft, target, eos, n_eos, ignore_eos,
                    batch, k, out);
}
