// Expert-parallel dispatch and combine over peer memory (NVLink 5 / NVSwitch).
//
// Every rank holds its own token rows (attention runs data-parallel) and E/world experts. One
// MoE layer call is:
//   1. ep_count        : per-expert assignment counts of the local rows.
//   2. ep_dispatch     : publishes the counts into every peer's count matrix (peer stores + flag),
//                        waits for all ranks' counts, derives every expert segment's offset on its
//                        owner (segments padded to 16 rows, sources in rank order), then scatters
//                        the token rows (read once per row, stored to each of its top-k owners) straight
//                        into the owners' expert input buffers with 16-byte peer stores; the last CTA flags "dispatch
//                        complete" to every peer. The owner's seg_off / counts arrays for the
//                        grouped GEMM are written by CTA 0 (no host involvement anywhere).
//   3. ep_wait         : the owner waits (bounded) until every source has flagged completion.
//   4. grouped GEMMs   : moe_grouped_gemm (moe.cu) on the received rows, gate/up + SwiGLU then down.
//   5. ep_combine      : flags "outputs ready", waits for every peer's flag, then each source row
//                        READS its k expert outputs directly from the owners' output buffers (peer
//                        loads) and sums them weighted, in ascending expert id, in FP32, one BF16
//                        rounding.
// The reference's only analogue is its 2-GPU "peer compute" hop, which bounces one layer's packet
// GPU0 -> pinned host -> GPU1 and back (src/backend/cuda/engine_moe.rs:1643-1830); its combine
// order contract (ascending expert id, kernels/moe_combine.cu:52-96) is kept.
//
// Arena layout (symmetric, identical on every rank), byte offsets in EpArena. All waits are
// bounded and report FF_ERR_TIMEOUT through the status word.
#include "comm.cuh"
#include "host_util.h"

namespace ff {

constexpr int EP_MAX_E = 512;
constexpr int EP_FLAG_COUNTS = 0, EP_FLAG_DISPATCH = 1, EP_FLAG_READY = 2;

struct EpArena {
  uint8_t* base[MAX_RANKS];
  int rank, world;
  int E, E_local;               // experts in total / per rank
  int hidden, capacity;         // row width, rows of the receive / output buffers
  long long off_flags;          // int32 [world][4]
  long long off_counts;         // int32 [world][E]
  long long off_x;              // bf16 [capacity][hidden]   (received token rows)
  long long off_y;              // bf16 [capacity][hidden]   (expert outputs, read by peers)
};

__device__ __forceinline__ int* ep_epoch(const EpArena& a) { return reinterpret_cast<int*>(a.base[a.rank]); }
__device__ __forceinline__ int* ep_done(const EpArena& a, int which) { return reinterpret_cast<int*>(a.base[a.rank]) + 1 + which; }
__device__ __forceinline__ int* ep_flag(const EpArena& a, int on_rank, int src, int which) {
  return reinterpret_cast<int*>(a.base[on_rank] + a.off_flags) + src * 4 + which;
}
__device__ __forceinline__ int* ep_counts(const EpArena& a, int on_rank, int src) {
  return reinterpret_cast<int*>(a.base[on_rank] + a.off_counts) + (size_t)src * a.E;
}

__global__ void ep_count_kernel(const int* __restrict__ ids, int n_assign, int E, int* __restrict__ counts, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_assign) return;
  const int e = ids[i];
  if (e < 0 || e >= E) { set_status(status, KID_MOE_DISPATCH, FF_ERR_BOUNDS, i, e); return; }
  atomicAdd(&counts[e], 1);
}

// grid: any number of CTAs (<= 1024), 256 threads. cursors: int32[E] zeroed before launch.
// pos: int32 [n_assign] = owner_rank * capacity + slot (or -1).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpArena a, const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                   const int* __restrict__ my_counts, int* __restrict__ cursors, int* __restrict__ pos, int rows,
                   int top_k, int ldx, int* __restrict__ seg_off_out, int* __restrict__ counts_out, int* status,
                   int row_vecs) {
  __shared__ int s_base[EP_MAX_E];     // first slot of (expert e, source = me) on the owner
  __shared__ int s_tot[EP_MAX_E];
  __shared__ int s_ok;
  const int epoch = ld_volatile(ep_epoch(a)) + 1;
  const int E = a.E, El = a.E_local;
  // 1. publish my counts (CTA 0) ------------------------------------------------------------
  if (blockIdx.x == 0) {
    for (int p = 0; p < a.world; ++p) {
      int* dst = ep_counts(a, p, a.rank);
      for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = my_counts[e];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_release_sys(ep_flag(a, p, a.rank, EP_FLAG_COUNTS), epoch);
    }
  }
  // 2. every CTA waits for all ranks' counts -------------------------------------------------
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world)
    if (!wait_flag(ep_flag(a, a.rank, threadIdx.x, EP_FLAG_COUNTS), epoch, status, KID_MOE_DISPATCH, threadIdx.x)) s_ok = 0;
  __syncthreads();
  if (!s_ok) return;
  // 3. offsets: thread e -> total over sources and the part before me ----------------------------
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int s = 0; s < a.world; ++s) {
      const int c = ld_volatile(ep_counts(a, a.rank, s) + e);
      tot += c;
      if (s < a.rank) before += c;
    }
    s_tot[e] = tot;
    s_base[e] = before;
  }
  __syncthreads();
  // exclusive scan of pad16(total) inside each owner's expert range (serial per owner: E_local small)
  if (threadIdx.x < a.world) {
    const int d = threadIdx.x;
    int run = 0;
    for (int le = 0; le < El; ++le) {
      const int e = d * El + le;
      const int t = s_tot[e];
      s_base[e] += run;
      if (d == a.rank && blockIdx.x == 0) { seg_off_out[le] = run; counts_out[le] = t; }
      run += ((t + 15) / 16) * 16;
    }
    if (d == a.rank && blockIdx.x == 0) seg_off_out[El] = run;
    if (run > a.capacity) set_status(status, KID_MOE_DISPATCH, FF_ERR_CAPACITY, run, a.capacity);
  }
  __syncthreads();
  // 4. scatter rows: one warp per token row. Lane j < top_k claims the slot of assignment j; the row is
  //    read once into registers (16 vectors per lane per pass) and stored to each of its k owners.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  // 16-byte vectors of a travelling row: hidden / 8 for BF16 rows; packed FP8 records ([codes | 1x128 scales]) are
  // about half of that
  const int nvec = row_vecs;
  for (int r = blockIdx.x * wpb + warp; r < rows; r += gridDim.x * wpb) {
    int slot = -1, d = 0;
    if (lane < top_k) {
      const int e = ids[(size_t)r * top_k + lane];
      if (e >= 0 && e < E) {
        d = e / El;
        slot = s_base[e] + atomicAdd(&cursors[e], 1);
        if (slot >= a.capacity) slot = -1;
      }
      pos[(size_t)r * top_k + lane] = slot < 0 ? -1 : d * a.capacity + slot;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r * ldx);
    for (int v0 = 0; v0 < nvec; v0 += 32 * 16) {
      uint4 reg[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int v = v0 + u * 32 + lane;
        if (v < nvec) reg[u] = __ldg(src + v);
      }
      for (int j = 0; j < top_k; ++j) {
        const int sj = __shfl_sync(0xffffffffu, slot, j), dj = __shfl_sync(0xffffffffu, d, j);
        if (sj < 0) continue;
        uint4* dst = reinterpret_cast<uint4*>(a.base[dj] + a.off_x) + (size_t)sj * nvec;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int v = v0 + u * 32 + lane;
          if (v < nvec) dst[v] = reg[u];
        }
      }
    }
  }
  // 5. completion: last CTA flags every peer -------------------------------------------------------
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(ep_done(a, 0), 1);
    if (prev == (int)gridDim.x - 1) {
      *ep_done(a, 0) = 0;
      __threadfence_system();
      for (int p = 0; p < a.world; ++p) st_release_sys(ep_flag(a, p, a.rank, EP_FLAG_DISPATCH), epoch);
    }
  }
}

__global__ void ep_wait_kernel(EpArena a, int which, int* status) {
  const int epoch = ld_volatile(ep_epoch(a)) + 1;
  if (threadIdx.x < a.world) wait_flag(ep_flag(a, a.rank, threadIdx.x, which), epoch, status, KID_MOE_DISPATCH, 16 + threadIdx.x);
}

// grid (rows), 256 threads.
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpArena a, const int* __restrict__ pos, const int* __restrict__ ids, const float* __restrict__ w,
                  __nv_bfloat16* __restrict__ out, int rows, int top_k, int* status) {
  const int epoch = ld_volatile(ep_epoch(a)) + 1;
  __shared__ int s_pos[16]; __shared__ float s_w[16]; __shared__ int s_ok;
  // outputs of my experts are complete (stream order): tell everyone, then wait for everyone
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int p = 0; p < a.world; ++p) st_release_sys(ep_flag(a, p, a.rank, EP_FLAG_READY), epoch);
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < a.world)
    if (!wait_flag(ep_flag(a, a.rank, threadIdx.x, EP_FLAG_READY), epoch, status, KID_MOE_COMBINE, threadIdx.x)) s_ok = 0;
  const int row = blockIdx.x;
  if (threadIdx.x == 32) {
    int idv[16], pv[16]; float wv[16];
    for (int j = 0; j < top_k; ++j) { idv[j] = ids[(size_t)row * top_k + j]; pv[j] = pos[(size_t)row * top_k + j]; wv[j] = w[(size_t)row * top_k + j]; }
    for (int i = 1; i < top_k; ++i) {
      const int iv = idv[i], pp = pv[i]; const float ww = wv[i];
      int b = i - 1;
      while (b >= 0 && idv[b] > iv) { idv[b + 1] = idv[b]; pv[b + 1] = pv[b]; wv[b + 1] = wv[b]; --b; }
      idv[b + 1] = iv; pv[b + 1] = pp; wv[b + 1] = ww;
    }
    for (int j = 0; j < top_k; ++j) { s_pos[j] = pv[j]; s_w[j] = wv[j]; }
  }
  __syncthreads();
  if (s_ok) {
    const int nvec = a.hidden >> 3;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      // all peer loads of a batch of 8 contributions are in flight before the first is used
      for (int j0 = 0; j0 < top_k; j0 += 8) {
        uint4 dd[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int p = j0 + u < top_k ? s_pos[j0 + u] : -1;
          dd[u] = make_uint4(0u, 0u, 0u, 0u);
          if (p >= 0) {
            const int d = p / a.capacity, slot = p - d * a.capacity;
            dd[u] = __ldcg(reinterpret_cast<const uint4*>(a.base[d] + a.off_y) + (size_t)slot * nvec + v);
          }
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (j0 + u >= top_k || s_pos[j0 + u] < 0) continue;
          const uint32_t* dp = reinterpret_cast<const uint32_t*>(&dd[u]);
          const float ww = s_w[j0 + u];
#pragma unroll
          for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(dp[i]); acc[2 * i] += ww * f.x; acc[2 * i + 1] += ww * f.y; }
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + (size_t)row * a.hidden)[v] = o;
    }
  }
  // the last CTA closes the layer call: every peer has read what it needs from me only after
  // ITS combine, which is ordered before its next dispatch, so publishing the epoch here is safe
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(ep_done(a, 1), 1);
    if (prev == (int)gridDim.x - 1) {
      *ep_done(a, 1) = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(ep_epoch(a)) = epoch;
    }
  }
}

}  // namespace ff
using namespace ff;

struct EpArenaHost {
  unsigned long long ptrs[8];
  int rank, world, E, E_local, hidden, capacity;
  long long off_flags, off_counts, off_x, off_y;
};

static int to_arena(const EpArenaHost* h, EpArena& a) {
  if (!h || h->world < 1 || h->world > MAX_RANKS || h->rank < 0 || h->rank >= h->world) return FF_HOST_BAD_SHAPE;
  if (h->E > EP_MAX_E || h->E != h->E_local * h->world || h->hidden % 8 || h->capacity % 16) return FF_HOST_BAD_SHAPE;
  for (int i = 0; i < MAX_RANKS; ++i) a.base[i] = i < h->world ? reinterpret_cast<uint8_t*>(h->ptrs[i]) : nullptr;
  a.rank = h->rank; a.world = h->world; a.E = h->E; a.E_local = h->E_local; a.hidden = h->hidden;
  a.capacity = h->capacity; a.off_flags = h->off_flags; a.off_counts = h->off_counts; a.off_x = h->off_x;
  a.off_y = h->off_y;
  return 0;
}

// Bytes of the symmetric arena for the given geometry and the offsets of its parts.
FF_EXPORT long long ff_ep_arena_layout(int world, int E, int hidden, int capacity, long long* off_flags,
                                       long long* off_counts, long long* off_x, long long* off_y) {
  long long o = 256;
  *off_flags = o; o += (long long)world * 4 * 4; o = (o + 255) / 256 * 256;
  *off_counts = o; o += (long long)world * E * 4; o = (o + 255) / 256 * 256;
  *off_x = o; o += (long long)capacity * hidden * 2; o = (o + 255) / 256 * 256;
  *off_y = o; o += (long long)capacity * hidden * 2; o = (o + 255) / 256 * 256;
  return o;
}

// counts_scratch / cursors: int32[E] each (device, local). seg_off_out: int32[E_local+1],
// counts_out: int32[E_local], pos: int32[rows*top_k].
static int ep_dispatch_launch(const EpArenaHost* h, const void* x, const int* ids, int rows, int top_k, int ldx,
                              int* counts_scratch, int* cursors, int* pos, int* seg_off_out, int* counts_out,
                              int* status, cudaStream_t s, int row_vecs) {
  EpArena a;
  if (int r = to_arena(h, a)) return r;
  if (rows <= 0 || top_k < 1 || top_k > 16 || ldx % 8) return FF_HOST_BAD_SHAPE;
  if (row_vecs <= 0 || row_vecs > (a.hidden >> 3) || ldx < row_vecs * 8) return FF_HOST_BAD_SHAPE;
  cudaError_t e = cudaMemsetAsync(counts_scratch, 0, (size_t)a.E * 4, s);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemsetAsync(cursors, 0, (size_t)a.E * 4, s);
  if (e != cudaSuccess) return (int)e;
  const int n = rows * top_k;
  ep_count_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, n, a.E, counts_scratch, status);
  int ctas = (rows + 7) / 8;
  if (ctas > 296) ctas = 296;
  if (ctas < 1) ctas = 1;
  ep_dispatch_kernel<<<ctas, 256, 0, s>>>(a, (const __nv_bfloat16*)x, ids, counts_scratch, cursors, pos, rows, top_k,
                                          ldx, seg_off_out, counts_out, status, row_vecs);
  ep_wait_kernel<<<1, 32, 0, s>>>(a, EP_FLAG_DISPATCH, status);
  return launch_result();
}

FF_EXPORT int ff_ep_dispatch(const EpArenaHost* h, const void* x, const int* ids, int rows, int top_k, int ldx,
                             int* counts_scratch, int* cursors, int* pos, int* seg_off_out, int* counts_out,
                             int* status, cudaStream_t s) {
  return ep_dispatch_launch(h, x, ids, rows, top_k, ldx, counts_scratch, cursors, pos, seg_off_out, counts_out, status, s,
                            h->hidden >> 3);
}

// Dispatch of packed records of `row_bytes` bytes (a multiple of 16, at most the arena's BF16 row): x rows are
// `ld_bytes` apart. The receive buffer then holds records `row_bytes` apart (slot s at off_x + s * row_bytes).
FF_EXPORT int ff_ep_dispatch_bytes(const EpArenaHost* h, const void* x, const int* ids, int rows, int top_k, int ld_bytes,
                                   int row_bytes, int* counts_scratch, int* cursors, int* pos, int* seg_off_out,
                                   int* counts_out, int* status, cudaStream_t s) {
  if (row_bytes <= 0 || row_bytes % 16 || ld_bytes % 16 || ld_bytes < row_bytes) return FF_HOST_BAD_SHAPE;
  return ep_dispatch_launch(h, x, ids, rows, top_k, ld_bytes / 2, counts_scratch, cursors, pos, seg_off_out, counts_out,
                            status, s, row_bytes / 16);
}

FF_EXPORT int ff_ep_combine(const EpArenaHost* h, const int* pos, const int* ids, const float* w, void* out, int rows,
                            int top_k, int* status, cudaStream_t s) {
  EpArena a;
  if (int r = to_arena(h, a)) return r;
  if (rows <= 0 || top_k < 1 || top_k > 16) return FF_HOST_BAD_SHAPE;
  ep_combine_kernel<<<rows, 256, 0, s>>>(a, pos, ids, w, (__nv_bfloat16*)out, rows, top_k, status);
  return launch_result();
}
