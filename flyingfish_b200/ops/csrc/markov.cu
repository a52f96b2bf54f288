// Markov head of the tree drafter: for every request p with parent token tok[p] and base-logit row B[row[p]],
//   bias[p][v] = bf16( w2[v] . w1[tok[p]] )            (K = 256; the decode GEMM of this library, BF16 output)
//   s[p][v]    = bf16( bias[p][v] + B[row[p]][v] )
//   top-4[p]   = the four largest s (strictly greater wins, ties to the smaller token id)
//   logp[p][j] = (s[top4 j] - m) - log(sum_v exp(s[v] - m)),  m = max_v s[v];  lse[p] = m + log(sum)
// This file holds the second half: the row-wise top-4 + log-sum-exp over the vocabulary, in two
// phases (vocab chunks of 4096 per CTA, then a merge in ascending chunk order), so a request's outputs do not
// depend on the batch it is in. Restates kernels/markov.cu of the reference (:1-55 contract), which computes the
// bias with mma.sync inside the same kernel over 256-row vocab blocks.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int MK_CHUNK = 4096;

struct Top4 { float s[4]; int id[4]; };

__device__ __forceinline__ bool mk_better(float s, int id, float s2, int id2) { return s > s2 || (s == s2 && id < id2); }
__device__ __forceinline__ void mk_offer(Top4& t, float s, int id) {
  if (!mk_better(s, id, t.s[3], t.id[3])) return;
  int j = 3;
  while (j > 0 && mk_better(s, id, t.s[j - 1], t.id[j - 1])) { t.s[j] = t.s[j - 1]; t.id[j] = t.id[j - 1]; --j; }
  t.s[j] = s; t.id[j] = id;
}
__device__ __forceinline__ void mk_merge_ml(float& m, float& l, float m2, float l2) {
  const float mn = fmaxf(m, m2);
  l = (m == -INFINITY ? 0.f : l * expf(m - mn)) + (m2 == -INFINITY ? 0.f : l2 * expf(m2 - mn));
  m = mn;
}

// grid (chunks, P), 256 threads. part_top [P][chunks][4] (score, id as float bits) x2, part_ml [P][chunks][2]
__global__ void __launch_bounds__(256)
markov_top4_phase1(const __nv_bfloat16* __restrict__ bias, const __nv_bfloat16* __restrict__ base,
                   const int* __restrict__ req_row, int V, int ld_bias, int ld_base, float* __restrict__ part_top,
                   float* __restrict__ part_ml) {
  pdl_trigger();
  pdl_wait();
  __shared__ float ss[256 * 4];
  __shared__ int sid[256 * 4];
  __shared__ float sm[256], sl[256];
  const int p = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x;
  const __nv_bfloat16* brow = bias + (size_t)p * ld_bias;
  const __nv_bfloat16* lrow = base + (size_t)req_row[p] * ld_base;
  Top4 t;
#pragma unroll
  for (int j = 0; j < 4; ++j) { t.s[j] = -INFINITY; t.id[j] = 0x7fffffff; }
  float m = -INFINITY, l = 0.f;
  const int v0 = chunk * MK_CHUNK, v1 = min(V, v0 + MK_CHUNK);
  for (int v = v0 + tid; v < v1; v += 256) {
    const float s = __bfloat162float(__float2bfloat16(__bfloat162float(brow[v]) + __bfloat162float(lrow[v])));
    mk_offer(t, s, v);
    if (s > m) { l = l * expf(m - s) + 1.f; m = s; } else { l += expf(s - m); }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) { ss[tid * 4 + j] = t.s[j]; sid[tid * 4 + j] = t.id[j]; }
  sm[tid] = m; sl[tid] = l;
  __syncthreads();
  for (int stride = 128; stride > 0; stride >>= 1) {
    if (tid < stride) {
      Top4 a;
#pragma unroll
      for (int j = 0; j < 4; ++j) { a.s[j] = ss[tid * 4 + j]; a.id[j] = sid[tid * 4 + j]; }
#pragma unroll
      for (int j = 0; j < 4; ++j) mk_offer(a, ss[(tid + stride) * 4 + j], sid[(tid + stride) * 4 + j]);
#pragma unroll
      for (int j = 0; j < 4; ++j) { ss[tid * 4 + j] = a.s[j]; sid[tid * 4 + j] = a.id[j]; }
      float mm = sm[tid], ll = sl[tid];
      mk_merge_ml(mm, ll, sm[tid + stride], sl[tid + stride]);
      sm[tid] = mm; sl[tid] = ll;
    }
    __syncthreads();
  }
  if (tid < 4) {
    const size_t at = ((size_t)p * gridDim.x + chunk) * 8 + tid * 2;
    part_top[at] = ss[tid]; part_top[at + 1] = __int_as_float(sid[tid]);
  }
  if (tid == 0) { part_ml[((size_t)p * gridDim.x + chunk) * 2] = sm[0]; part_ml[((size_t)p * gridDim.x + chunk) * 2 + 1] = sl[0]; }
}

// grid P, 32 threads
__global__ void markov_top4_phase2(const float* __restrict__ part_top, const float* __restrict__ part_ml, int chunks,
                                   int* __restrict__ top4, float* __restrict__ logp, float* __restrict__ lse) {
  pdl_trigger();
  pdl_wait();
  if (threadIdx.x != 0) return;
  const int p = blockIdx.x;
  Top4 t;
  for (int j = 0; j < 4; ++j) { t.s[j] = -INFINITY; t.id[j] = 0x7fffffff; }
  float m = -INFINITY, l = 0.f;
  for (int c = 0; c < chunks; ++c) {
    const float* pt = part_top + ((size_t)p * chunks + c) * 8;
    for (int j = 0; j < 4; ++j) mk_offer(t, pt[2 * j], __float_as_int(pt[2 * j + 1]));
    mk_merge_ml(m, l, part_ml[((size_t)p * chunks + c) * 2], part_ml[((size_t)p * chunks + c) * 2 + 1]);
  }
  const float logsum = logf(l);
  for (int j = 0; j < 4; ++j) { top4[p * 4 + j] = t.id[j]; logp[p * 4 + j] = (t.s[j] - m) - logsum; }
  lse[p] = m + logsum;
}

}  // namespace ff
using namespace ff;

// bias [P, ld_bias] bf16, base [rows, ld_base] bf16, req_row [P]; scratch: part_top [P*chunks*8] f32, part_ml [P*chunks*2]
FF_EXPORT int ff_markov_top4(const void* bias, const void* base, const int* req_row, int P, int V, int ld_bias, int ld_base,
                             float* part_top, float* part_ml, int* top4, float* logp, float* lse, cudaStream_t s) {
  if (P <= 0 || V < 4) return FF_HOST_BAD_SHAPE;
  const int chunks = (V + MK_CHUNK - 1) / MK_CHUNK;
  if (int lr = launch_pdl(markov_top4_phase1, dim3(chunks, P), dim3(256), 0, s, 0, (const __nv_bfloat16*)bias,
                          (const __nv_bfloat16*)base, req_row, V, ld_bias, ld_base, part_top, part_ml)) return lr;
  if (int lr = launch_pdl(markov_top4_phase2, dim3(P), dim3(32), 0, s, 0, (const float*)part_top, (const float*)part_ml, chunks,
                          top4, logp, lse)) return lr;
  return launch_result();
}
