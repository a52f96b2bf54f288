// DSA: top-k sparse attention support kernels (GLM-style indexer).
//
// Every cached token carries a latent row (the attention key/value) and an index row: a 128-dim index
// key and a 128-dim pooling logit. Four consecutive tokens form a pool: per channel, a soft-max over the
// four (logit + position embedding) weights the four index keys into one pooled key. A query scores
// every complete pool that ends at or before its position with 32 index heads,
//     score = sum_h relu(q_h . k_pool / sqrt(128)) * w_h / sqrt(32),
// keeps the top 512 pools, expands them to token indices (4 per pool) plus the tokens after the last
// complete pool, and attends sparsely over those latent rows (csrc/latent.cu, gathered form).
// Restates kernels/dsa.cu of the reference (:99-144 pooling with BF16-rounded probabilities and
// products, :146-233 index scores + top-k, :235-294 expansion) for batches of sequences stored
// contiguously; the reference's top-k is a single-thread bounded heap (kernels/dsa_topk.cuh), here a
// block-wide radix select picks the k-th score, ties go to the lower pool id, and the winners are
// sorted by (score descending, id ascending) with a bitonic network.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

constexpr int DSA_DIM = 128;       // index key / logit width
constexpr int DSA_POOL = 4;
constexpr int DSA_HEADS = 32;
constexpr int DSA_MAXK = 512;

__device__ __forceinline__ float dsa_bf16r(float x) { return __bfloat162float(__float2bfloat16(x)); }

// idx_key / pool_logit [tokens, 128] bf16 (contiguous per sequence, sequence s starts at seq_start[s] and has
// seq_len[s] tokens), ape [4, 128] bf16 -> pooled [pools_total, 128] bf16 where sequence s owns pools
// pool_start[s] .. pool_start[s] + seq_len[s] / 4. grid (max pools per sequence, sequences), 128 threads.
__global__ void dsa_pool_kernel(const __nv_bfloat16* __restrict__ idx_key, const __nv_bfloat16* __restrict__ pool_logit,
                                const __nv_bfloat16* __restrict__ ape, const int* __restrict__ seq_start,
                                const int* __restrict__ seq_len, const int* __restrict__ pool_start,
                                __nv_bfloat16* __restrict__ pooled) {
  pdl_trigger();
  pdl_wait();
  const int s = blockIdx.y, pool = blockIdx.x, ch = threadIdx.x;
  if (pool >= seq_len[s] / DSA_POOL) return;
  const size_t t0 = (size_t)seq_start[s] + (size_t)pool * DSA_POOL;
  float lg[DSA_POOL], ky[DSA_POOL], mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < DSA_POOL; ++j) {
    lg[j] = __bfloat162float(pool_logit[(t0 + j) * DSA_DIM + ch]) + __bfloat162float(ape[j * DSA_DIM + ch]);
    ky[j] = __bfloat162float(idx_key[(t0 + j) * DSA_DIM + ch]);
    mx = fmaxf(mx, lg[j]);
  }
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < DSA_POOL; ++j) { lg[j] = expf(lg[j] - mx); sum += lg[j]; }
  float v = 0.f;
#pragma unroll
  for (int j = 0; j < DSA_POOL; ++j) v += dsa_bf16r(dsa_bf16r(lg[j] / sum) * ky[j]);
  pooled[((size_t)pool_start[s] + pool) * DSA_DIM + ch] = __float2bfloat16(v);
}

// scores[r, p] for p < n_cand[r]: q [rows, 32, 128] bf16, w [rows, 32] bf16, pooled rows of the row's sequence
// start at pool_base[r]. grid (ceil(max_cand / 64), rows), 256 threads: a warp scores 8 pools.
__global__ void __launch_bounds__(256)
dsa_index_score_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ pooled, const int* __restrict__ pool_base,
                       const int* __restrict__ n_cand, float* __restrict__ scores, int ld_scores) {
  pdl_trigger();
  pdl_wait();
  __shared__ float sq[DSA_HEADS * DSA_DIM];
  __shared__ float sw[DSA_HEADS];
  const int r = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = n_cand[r];
  if ((int)blockIdx.x * 64 >= n) return;
  for (int i = tid; i < DSA_HEADS * DSA_DIM; i += 256) sq[i] = __bfloat162float(q[(size_t)r * DSA_HEADS * DSA_DIM + i]);
  if (tid < DSA_HEADS) sw[tid] = __bfloat162float(w[(size_t)r * DSA_HEADS + tid]) * 0.1767766922712326f;
  __syncthreads();
  for (int i = 0; i < 8; ++i) {
    const int p = blockIdx.x * 64 + warp * 8 + i;
    if (p >= n) break;
    const __nv_bfloat16* kp = pooled + ((size_t)pool_base[r] + p) * DSA_DIM;
    float k4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) k4[j] = __bfloat162float(kp[lane + 32 * j]);
    float score = 0.f;
    for (int h = 0; h < DSA_HEADS; ++h) {
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) dot = fmaf(sq[h * DSA_DIM + lane + 32 * j], k4[j], dot);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      score += fmaxf(dot * 0.0883883461356163f, 0.f) * sw[h];
    }
    if (lane == 0) scores[(size_t)r * ld_scores + p] = score;
  }
}

// order-preserving map float -> uint32 (larger float = larger key); scores are finite
__device__ __forceinline__ uint32_t dsa_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Top-k of scores[r, 0..n): selected [rows, k] ids (score descending, ties by lower id, -1 padded),
// sel_scores [rows, k]. One block of 1024 threads per row; k <= 512.
__global__ void __launch_bounds__(1024)
dsa_topk_kernel(const float* __restrict__ scores, const int* __restrict__ n_cand, int ld_scores, int k,
                int* __restrict__ selected, float* __restrict__ sel_scores) {
  pdl_trigger();
  pdl_wait();
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_remaining, s_count_gt, s_tie_base;
  __shared__ int s_scan[1024];
  __shared__ uint32_t sk[DSA_MAXK];      // keys of the winners
  __shared__ int si[DSA_MAXK];           // their ids
  const int r = blockIdx.x, tid = threadIdx.x;
  const int n = n_cand[r];
  const float* sc = scores + (size_t)r * ld_scores;
  const int keep = min(k, n);
  for (int i = tid; i < DSA_MAXK; i += 1024) { sk[i] = 0u; si[i] = 0x7fffffff; }
  if (tid == 0) { s_prefix = 0u; s_mask = 0u; s_remaining = keep; s_count_gt = 0; }
  __syncthreads();
  if (keep > 0) {
    // radix select of the keep-th largest key, one byte per pass from the top
    for (int pass = 3; pass >= 0; --pass) {
      for (int i = tid; i < 256; i += 1024) hist[i] = 0;
      __syncthreads();
      const uint32_t prefix = s_prefix, mask = s_mask;
      for (int i = tid; i < n; i += 1024) {
        const uint32_t key = dsa_key(sc[i]);
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> (8 * pass)) & 255u], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int rem = s_remaining, bin = 255;
        for (; bin > 0; --bin) { if (hist[bin] >= rem) break; rem -= hist[bin]; }
        s_remaining = rem;                                   // rank of the k-th key inside the chosen bin
        s_prefix = prefix | ((uint32_t)bin << (8 * pass));
        s_mask = mask | (255u << (8 * pass));
      }
      __syncthreads();
    }
    const uint32_t kth = s_prefix;
    const int ties_wanted = s_remaining;                     // how many keys equal to kth are kept (lowest ids)
    // winners above the threshold (any order), then the ties in id order through a block scan
    for (int base = 0; base < n; base += 1024) {
      const int i = base + tid;
      if (i < n && dsa_key(sc[i]) > kth) { const int at = atomicAdd(&s_count_gt, 1); sk[at] = dsa_key(sc[i]); si[at] = i; }
    }
    __syncthreads();
    if (tid == 0) s_tie_base = 0;
    __syncthreads();
    const int gt = s_count_gt;
    for (int base = 0; base < n; base += 1024) {
      const int i = base + tid;
      const int flag = (i < n && dsa_key(sc[i]) == kth) ? 1 : 0;
      s_scan[tid] = flag;
      __syncthreads();
      for (int off = 1; off < 1024; off <<= 1) {             // inclusive scan
        const int v = (tid >= off) ? s_scan[tid - off] : 0;
        __syncthreads();
        s_scan[tid] += v;
        __syncthreads();
      }
      const int rank = s_tie_base + s_scan[tid] - flag;      // ties before this one, in id order
      if (flag && rank < ties_wanted) { sk[gt + rank] = kth; si[gt + rank] = i; }
      __syncthreads();
      if (tid == 1023) s_tie_base += s_scan[1023];
      __syncthreads();
    }
    // bitonic sort of the 512 slots by (key descending, id ascending); empty slots have key 0, id INT_MAX
    for (int size = 2; size <= DSA_MAXK; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        if (tid < DSA_MAXK / 2) {
          const int lo = 2 * tid - (tid & (stride - 1)), hi = lo + stride;
          const bool desc = ((lo & size) == 0);
          const uint32_t ka = sk[lo], kb = sk[hi]; const int ia = si[lo], ib = si[hi];
          const bool a_first = (ka > kb) || (ka == kb && ia < ib);     // a precedes b in the wanted order
          if (a_first != desc) { sk[lo] = kb; sk[hi] = ka; si[lo] = ib; si[hi] = ia; }
        }
        __syncthreads();
      }
    }
  }
  for (int i = tid; i < k; i += 1024) {
    const bool live = i < keep;
    selected[(size_t)r * k + i] = live ? si[i] : -1;
    sel_scores[(size_t)r * k + i] = live ? sc[si[i]] : -INFINITY;
  }
}

// Token indices of a selection: indices [rows, k*4 + 3]. Row r of sequence with first token seq_base[r] sees
// tokens up to position pos[r] (inclusive, sequence-local): the 4 tokens of every selected pool, then the
// tokens after the last complete pool that ends <= pos. Unused entries are -1. Indices are global rows.
__global__ void dsa_expand_kernel(const int* __restrict__ selected, const int* __restrict__ seq_base,
                                  const int* __restrict__ pos, int k, int* __restrict__ indices) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x, width = k * DSA_POOL + DSA_POOL - 1;
  const int npools = (pos[r] + 1) / DSA_POOL;                 // complete pools ending at or before pos
  const int tail0 = npools * DSA_POOL, ntail = pos[r] + 1 - tail0;
  const int nsel = min(k, npools);
  for (int slot = threadIdx.x; slot < width; slot += blockDim.x) {
    int idx = -1;
    if (slot < nsel * DSA_POOL) {
      const int pool = selected[(size_t)r * k + slot / DSA_POOL];
      if (pool >= 0) idx = seq_base[r] + pool * DSA_POOL + slot % DSA_POOL;
    } else if (slot - nsel * DSA_POOL < ntail) {
      idx = seq_base[r] + tail0 + slot - nsel * DSA_POOL;
    }
    indices[(size_t)r * width + slot] = idx;
  }
}

// Checkpoint of per-token state rows for speculative rollback: save (RESTORE = false) or put back the rows
// `rows[0 .. n)` of every state table (latent rows, index keys, pooling logits, pooled keys: one base pointer and one
// row size per table) in a single launch. snapshot layout: [table][n][max_vecs] 16-byte vectors. grid (n, tables).
// The counterpart of the reference's dsa_checkpoint (kernels/dsa.cu:427-481), which saves and restores the ring slots a
// draft round overwrites; here the tables are addressed by global row.
template <bool RESTORE>
__global__ void dsa_checkpoint_kernel(const unsigned long long* __restrict__ tables, const int* __restrict__ row_vecs,
                                      const int* __restrict__ table_rows, const int* __restrict__ rows,
                                      uint4* __restrict__ snap, int max_vecs, int* status) {
  pdl_trigger();
  pdl_wait();
  const int j = blockIdx.x, c = blockIdx.y;
  const int r = rows[j];
  if (r < 0 || r >= table_rows[c]) { if (threadIdx.x == 0) set_status(status, KID_DSA, FF_ERR_BOUNDS, j, r); return; }
  const int nv = row_vecs[c];
  uint4* base = reinterpret_cast<uint4*>(tables[c]) + (size_t)r * nv;
  uint4* sn = snap + ((size_t)c * gridDim.x + j) * max_vecs;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    if (RESTORE) base[i] = sn[i]; else sn[i] = base[i];
  }
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_dsa_pool(const void* idx_key, const void* pool_logit, const void* ape, const int* seq_start,
                          const int* seq_len, const int* pool_start, void* pooled, int sequences, int max_pools,
                          cudaStream_t s) {
  if (sequences <= 0 || max_pools <= 0) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(dsa_pool_kernel, dim3(max_pools, sequences), dim3(DSA_DIM), 0, s, 0, (const __nv_bfloat16*)idx_key,
                          (const __nv_bfloat16*)pool_logit, (const __nv_bfloat16*)ape, seq_start, seq_len, pool_start,
                          (__nv_bfloat16*)pooled)) return lr;
  return launch_result();
}

// scores [rows, ld_scores] f32 scratch; selected / sel_scores [rows, k]
FF_EXPORT int ff_dsa_index_topk(const void* q, const void* w, const void* pooled, const int* pool_base, const int* n_cand,
                                float* scores, int ld_scores, int rows, int max_cand, int k, int* selected,
                                float* sel_scores, cudaStream_t s) {
  if (rows <= 0 || max_cand < 0 || k <= 0 || k > DSA_MAXK || ld_scores < max_cand) return FF_HOST_BAD_SHAPE;
  if (max_cand > 0) {
    if (int lr = launch_pdl(dsa_index_score_kernel, dim3((max_cand + 63) / 64, rows), dim3(256), 0, s, 0,
                            (const __nv_bfloat16*)q, (const __nv_bfloat16*)w, (const __nv_bfloat16*)pooled, pool_base, n_cand,
                            scores, ld_scores)) return lr;
  }
  if (int lr = launch_pdl(dsa_topk_kernel, dim3(rows), dim3(1024), 0, s, 0, (const float*)scores, n_cand, ld_scores, k,
                          selected, sel_scores)) return lr;
  return launch_result();
}

FF_EXPORT int ff_dsa_expand(const int* selected, const int* seq_base, const int* pos, int rows, int k, int* indices,
                            cudaStream_t s) {
  if (rows <= 0 || k <= 0 || k > DSA_MAXK) return FF_HOST_BAD_SHAPE;
  if (int lr = launch_pdl(dsa_expand_kernel, dim3(rows), dim3(128), 0, s, 0, selected, seq_base, pos, k, indices)) return lr;
  return launch_result();
}

// tables / row_vecs / table_rows: device arrays of `n_tables` entries (base pointer, 16-byte vectors per row, rows in
// the table); rows: device int32[n]; snapshot: n_tables * n * max_vecs * 16 bytes.
FF_EXPORT int ff_dsa_checkpoint(const unsigned long long* tables, const int* row_vecs, const int* table_rows, int n_tables,
                                const int* rows, int n, void* snapshot, int max_vecs, int restore, int* status,
                                cudaStream_t s) {
  if (n_tables <= 0 || n <= 0 || max_vecs <= 0) return FF_HOST_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(snapshot) & 15) return FF_HOST_BAD_ALIGN;
  dim3 grid(n, n_tables);
  const int threads = max_vecs >= 128 ? 128 : 32;
  if (restore)
    return launch_pdl(dsa_checkpoint_kernel<true>, grid, dim3(threads), 0, s, 0, tables, row_vecs, table_rows, rows,
                      static_cast<uint4*>(snapshot), max_vecs, status);
  return launch_pdl(dsa_checkpoint_kernel<false>, grid, dim3(threads), 0, s, 0, tables, row_vecs, table_rows, rows,
                    static_cast<uint4*>(snapshot), max_vecs, status);
}
