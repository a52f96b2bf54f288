// Mixture-of-experts operators.
//   moe_topk      : scores + deterministic top-k from router logits (softmax / sigmoid / grouped
//                   "noaux" selection with bias), ties -> lower expert id, FP32 weights
//   moe_count / moe_scan_permute : per-expert counts, 16-row padded segment offsets and the gather
//                   of token rows into expert order -- all on the device, no host read-back
//                   (the reference syncs the counts to the host before its grouped GEMM,
//                   src/backend/cuda/moe/prefill.rs:1137)
//   moe_grouped_gemm : Y[seg rows, N] = Xsorted[seg rows, K] · W[e][N, K]ᵀ for every expert segment,
//                   swap-AB on tcgen05 (a 128-row slice of the expert weight is the UMMA A operand,
//                   up to 256 tokens of the segment are the UMMA N dimension), optional SwiGLU
//                   epilogue for gate/up weights interleaved per 64 rows
//   moe_combine   : FP32 sum of a row's k contributions in ascending expert id, one BF16 rounding
// Semantics follow kernels/moe_route.cu:1-30,155-390, kernels/moe_prefill.cu and
// kernels/moe_combine.cu:1-96 of the reference.
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

// ---------------------------------------------------------------------------------------
// routing: one warp per row, scores in shared memory
// score_mode: 0 softmax, 1 sigmoid, 2 noaux (sigmoid + bias for selection, groups), 3 as 2 with sqrt(softplus(x)) scores
// ---------------------------------------------------------------------------------------
constexpr int ROUTE_WARPS = 4;
constexpr int ROUTE_MAX_E = 512;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_topk_kernel(const __nv_bfloat16* __restrict__ logits, const float* __restrict__ bias, float* __restrict__ out_w,
                int* __restrict__ out_ids, int rows, int E, int top_k, int score_mode, int n_groups, int topk_groups,
                float routed_scaling, int renormalize, int ld, int* status) {
  __shared__ float s_score[ROUTE_WARPS][ROUTE_MAX_E];   // unbiased score
  __shared__ float s_sel[ROUTE_WARPS][ROUTE_MAX_E];     // selection score
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROUTE_WARPS + warp;
  if (row >= rows) return;
  float* sc = s_score[warp];
  float* sel = s_sel[warp];
  const __nv_bfloat16* lg = logits + (size_t)row * ld;
  if (score_mode == 0) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, __bfloat162float(lg[e]));
    mx = warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { const float v = expf(__bfloat162float(lg[e]) - mx); sc[e] = v; sum += v; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) { sc[e] *= inv; sel[e] = sc[e]; }
  } else {
    for (int e = lane; e < E; e += 32) {
      const float x = __bfloat162float(lg[e]);
      const float v = (score_mode == 3) ? sqrtf(x > 20.f ? x : log1pf(expf(x))) : 1.0f / (1.0f + expf(-x));
      sc[e] = v;
      sel[e] = (score_mode >= 2 && bias) ? v + bias[e] : v;
    }
  }
  __syncwarp();
  if (score_mode >= 2 && n_groups > 1) {
    const int gsz = E / n_groups;
    // group score = sum of the two best selection scores of the group
    float gscore = -INFINITY;
    if (lane < n_groups) {
      float b0 = -INFINITY, b1 = -INFINITY;
      for (int j = 0; j < gsz; ++j) {
        const float v = sel[lane * gsz + j];
        if (v > b0) { b1 = b0; b0 = v; } else if (v > b1) { b1 = v; }
      }
      gscore = b0 + b1;
    }
    unsigned keep = 0;
    for (int it = 0; it < topk_groups; ++it) {
      float v = (lane < n_groups && !((keep >> lane) & 1u)) ? gscore : -INFINITY;
      int i = lane;
      warp_argmax(v, i);
      keep |= 1u << i;
    }
    for (int e = lane; e < E; e += 32) if (!((keep >> (e / gsz)) & 1u)) sel[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.f;
  float my_w = 0.f; int my_id = 0;     // lane j keeps the j-th selection
  for (int it = 0; it < top_k; ++it) {
    float v = -INFINITY; int i = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float s = sel[e];
      if (s > v || (s == v && e < i)) { v = s; i = e; }
    }
    warp_argmax(v, i);
    if (i == 0x7fffffff || i >= E) { i = 0; if (lane == 0) set_status(status, KID_MOE_ROUTE, FF_ERR_NONFINITE, row, it); }
    const float w = sc[i];
    wsum += w;
    if (lane == it) { my_w = w; my_id = i; }
    __syncwarp();
    if (lane == 0) sel[i] = -INFINITY;
    __syncwarp();
  }
  if (lane < top_k) {
    float w = my_w;
    if (renormalize) w = w / fmaxf(wsum, 1e-20f);
    out_w[(size_t)row * top_k + lane] = w * routed_scaling;
    out_ids[(size_t)row * top_k + lane] = my_id;
  }
}

// ---------------------------------------------------------------------------------------
// count / scan / permute
// ---------------------------------------------------------------------------------------
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_assign, int E, int e_lo, int e_hi,
                                 int* __restrict__ counts, int* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_assign) return;
  const int e = ids[i];
  if (e == -1) return;                       // assignment served elsewhere (another tier / rank)
  if (e < 0 || e >= E) { set_status(status, KID_MOE_DISPATCH, FF_ERR_BOUNDS, i, e); return; }
  if (e >= e_lo && e < e_hi) atomicAdd(&counts[e - e_lo], 1);
}

// One block: seg_off[e] = sum of pad16(count) over earlier experts; cursors zeroed; total rows
// (padded) written to seg_off[E_local]. capacity = rows the sorted buffer can hold.
__global__ void __launch_bounds__(1024)
moe_scan_kernel(const int* __restrict__ counts, int* __restrict__ seg_off, int* __restrict__ cursors, int E_local,
                int capacity, int* status) {
  __shared__ int s[1024];
  const int t = threadIdx.x;
  const int c = t < E_local ? ((counts[t] + 15) / 16) * 16 : 0;
  s[t] = c;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = t >= o ? s[t - o] : 0;
    __syncthreads();
    s[t] += v;
    __syncthreads();
  }
  if (t < E_local) { seg_off[t] = s[t] - c; cursors[t] = 0; }
  if (t == E_local - 1) {
    seg_off[E_local] = s[t];
    if (s[t] > capacity) set_status(status, KID_MOE_DISPATCH, FF_ERR_CAPACITY, s[t], capacity);
  }
}

// one block per assignment (row, j): claim a slot in the expert's segment, copy the token row
__global__ void __launch_bounds__(128)
moe_permute_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, const int* __restrict__ seg_off,
                   int* __restrict__ cursors, __nv_bfloat16* __restrict__ sorted, int* __restrict__ pos, int hidden,
                   int top_k, int e_lo, int e_hi, int capacity, int ldx) {
  const int a = blockIdx.x;
  const int e = ids[a];
  __shared__ int slot_s;
  if (e < e_lo || e >= e_hi) { if (threadIdx.x == 0) pos[a] = -1; return; }
  if (threadIdx.x == 0) slot_s = seg_off[e - e_lo] + atomicAdd(&cursors[e - e_lo], 1);
  __syncthreads();
  const int slot = slot_s;
  if (threadIdx.x == 0) pos[a] = slot < capacity ? slot : -1;
  if (slot >= capacity) return;
  const int row = a / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint4* dst = reinterpret_cast<uint4*>(sorted + (size_t)slot * hidden);
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) dst[v] = src[v];
}

// ---------------------------------------------------------------------------------------
// grouped GEMM (swap-AB). grid (n_tiles, E_local). 192 threads.
//   W      : [E_local * Nw, K] bf16 (expert e rows at e*Nw)
//   Xs     : sorted tokens [capacity, K]; tensor map box = 16 rows x 64
//   Y      : [capacity, Nout] bf16; Nout = Nw (epi 0) or Nw/2 (epi 1: gate/up interleaved per 64
//            rows -> a 128-row tile holds 64 gate rows then the matching 64 up rows)
// ---------------------------------------------------------------------------------------
constexpr int GBM = 128, GBK = 64, G_STAGES_MAX = 8, G_TOK = 256;

struct alignas(8) GroupBars {
  uint64_t full[G_STAGES_MAX];
  uint64_t empty[G_STAGES_MAX];
  uint64_t tmem_full;
  uint64_t tmem_empty;
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ float silu_g(float x) { return x / (1.0f + __expf(-x)); }
__device__ __forceinline__ float bfr(float x) { return __bfloat162float(__float2bfloat16(x)); }

__global__ void __launch_bounds__(192, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                        __nv_bfloat16* __restrict__ Y, const int* __restrict__ seg_off, const int* __restrict__ counts,
                        int Nw, int K, int ldy, int epi, int pipe_bytes, int stage_off, int* status, int capacity) {
  int stages;
  extern __shared__ uint8_t smem_raw[];
  __shared__ GroupBars bars;
  const int e = blockIdx.y, tn = blockIdx.x;
  // a segment reaching past the row buffers (an overflowed dispatch, reported through the status word) is cut there
  const int cnt = min(counts[e], capacity - seg_off[e]);
  if (cnt <= 0) return;                                   // uniform for the CTA
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sT = reinterpret_cast<float*>(smem);             // staging [tok chunk of 64][128] fp32 = 32 KiB
  uint8_t* pipe = smem + stage_off;
  constexpr int A_BYTES = GBM * GBK * 2;
  // the token operand of a stage is sized for this expert's largest chunk, so experts with few
  // tokens (decode) get a deep weight pipeline out of the same shared memory
  const int ntok_max = min(G_TOK, ((cnt + 15) / 16) * 16);
  const int STAGE_BYTES = A_BYTES + ntok_max * GBK * 2;
  stages = min(G_STAGES_MAX, pipe_bytes / STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = seg_off[e];
  const int kblocks = (K + GBK - 1) / GBK;
  const int chunks = (cnt + G_TOK - 1) / G_TOK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < stages; ++i) { mbar_init(&bars.full[i], 1); mbar_init(&bars.empty[i], 1); }
    mbar_init(&bars.tmem_full, 1); mbar_init(&bars.tmem_empty, 4);
    bars.abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars.tmem_base, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars.tmem_base;
  volatile int* abort_flag = &bars.abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW); tma_prefetch_desc(&tmX);
      uint32_t it = 0; bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(G_TOK, ((cnt - c * G_TOK + 15) / 16) * 16);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.empty[s], ph ^ 1, abort_flag, status, KID_MOE_GEMM, 1)) { ok = false; break; }
          mbar_expect_tx(&bars.full[s], A_BYTES + ntok * GBK * 2);
          uint8_t* sa = pipe + s * STAGE_BYTES;
          tma_load_2d(sa, &tmW, &bars.full[s], kb * GBK, e * Nw + tn * GBM);
          for (int r = 0; r < ntok; r += 16)
            tma_load_2d(sa + A_BYTES + r * GBK * 2, &tmX, &bars.full[s], kb * GBK, row0 + c * G_TOK + r);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0; bool ok = true;
      for (int c = 0; c < chunks && ok; ++c) {
        const int ntok = min(G_TOK, ((cnt - c * G_TOK + 15) / 16) * 16);
        const uint32_t idesc = umma_idesc(1, 1, 0, 0, GBM, ntok);
        if (!mbar_wait(&bars.tmem_empty, (c & 1) ^ 1, abort_flag, status, KID_MOE_GEMM, 2)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % stages; const uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars.full[s], ph, abort_flag, status, KID_MOE_GEMM, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(pipe + s * STAGE_BYTES);
          const uint64_t da = umma_desc_sw128(sa, 16, 1024);
          const uint64_t db = umma_desc_sw128(sa + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < GBK / 16; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
          umma_commit(&bars.empty[s]);
        }
        if (ok) umma_commit(&bars.tmem_full);
      }
    }
  } else {
    const int q = warp & 3;
    const int nl = q * 32 + lane;
    const int ee = (warp - 2) * 32 + lane;
    bool ok = true;
    for (int c = 0; c < chunks && ok; ++c) {
      const int ntok = min(G_TOK, ((cnt - c * G_TOK + 15) / 16) * 16);
      const int real = min(G_TOK, cnt - c * G_TOK);
      if (!mbar_wait(&bars.tmem_full, c & 1, abort_flag, status, KID_MOE_GEMM, 4)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16);
      // process the chunk in sub-chunks of 64 tokens through the FP32 staging tile
      for (int t0 = 0; t0 < ntok; t0 += 64) {
        const int tcount = min(64, ntok - t0);
        for (int cc = 0; cc < tcount; cc += 16) {
          uint32_t r[16];
          tmem_ld_x16(taddr + t0 + cc, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) sT[(cc + j) * GBM + nl] = __uint_as_float(r[j]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int grow0 = row0 + c * G_TOK + t0;
        if (epi == 1) {
          // 64 outputs per tile: out[j] = bf16(silu(bf16 g)) * bf16(u), 8 threads per row (8 cols each)
          const int c8 = ee & 7, r0 = ee >> 3;            // 16 rows per pass
          for (int t = r0; t < tcount; t += 16) {
            if (t0 + t < real) {
              uint32_t o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int col = c8 * 8 + 2 * j;
                const float g0 = bfr(sT[t * GBM + col]), g1 = bfr(sT[t * GBM + col + 1]);
                const float u0 = bfr(sT[t * GBM + 64 + col]), u1 = bfr(sT[t * GBM + 64 + col + 1]);
                o[j] = pack_bf16x2(bfr(silu_g(g0)) * u0, bfr(silu_g(g1)) * u1);
              }
              *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t) * ldy + tn * 64 + c8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        } else {
          const int c16 = ee & 15, r0 = ee >> 4;          // 8 rows per pass, 8 cols per thread
          const int col = tn * GBM + c16 * 8;
          if (col < Nw) {
            for (int t = r0; t < tcount; t += 8) {
              if (t0 + t < real) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) o[j] = pack_bf16x2(sT[t * GBM + c16 * 8 + 2 * j], sT[t * GBM + c16 * 8 + 2 * j + 1]);
                *reinterpret_cast<uint4*>(Y + (size_t)(grow0 + t) * ldy + col) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tmem_empty);
    }
  }
  __syncthreads();
  if (bars.abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) { __nanosleep(1000); }
  }
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ---------------------------------------------------------------------------------------
// combine: out[row] = bf16( sum_j w[row,j] * y[pos[row,j]] ) in ascending expert id
// (+ optional residual-style accumulate into `out` when accumulate != 0). pos < 0 skips
// (assignment owned by another rank).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos, const int* __restrict__ ids,
                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int hidden, int top_k, int ldy,
                   int accumulate) {
  const int row = blockIdx.x;
  __shared__ int s_pos[16]; __shared__ float s_w[16];
  if (threadIdx.x == 0) {
    // insertion sort of the k choices by expert id (k <= 16)
    int idv[16], pv[16]; float wv[16];
    for (int j = 0; j < top_k; ++j) { idv[j] = ids[(size_t)row * top_k + j]; pv[j] = pos[(size_t)row * top_k + j]; wv[j] = w[(size_t)row * top_k + j]; }
    for (int a = 1; a < top_k; ++a) {
      const int iv = idv[a], pp = pv[a]; const float ww = wv[a];
      int b = a - 1;
      while (b >= 0 && idv[b] > iv) { idv[b + 1] = idv[b]; pv[b + 1] = pv[b]; wv[b + 1] = wv[b]; --b; }
      idv[b + 1] = iv; pv[b + 1] = pp; wv[b + 1] = ww;
    }
    for (int j = 0; j < top_k; ++j) { s_pos[j] = pv[j]; s_w[j] = wv[j]; }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < hidden / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int j = 0; j < top_k; ++j) {
      const int p = s_pos[j];
      if (p < 0) continue;
      const uint4 d = reinterpret_cast<const uint4*>(y + (size_t)p * ldy)[v];
      const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
      const float ww = s_w[j];
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(dp[i]); acc[2 * i] += ww * f.x; acc[2 * i + 1] += ww * f.y; }
    }
    uint4 o;
    if (accumulate) {
      const uint4 prev = reinterpret_cast<const uint4*>(out + (size_t)row * hidden)[v];
      const uint32_t* pp = reinterpret_cast<const uint32_t*>(&prev);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = unpack_bf16x2(pp[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
    }
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (size_t)row * hidden)[v] = o;
  }
}

}  // namespace ff
using namespace ff;

FF_EXPORT int ff_moe_topk(const void* logits, const float* bias, float* out_w, int* out_ids, int rows, int E,
                          int top_k, int score_mode, int n_groups, int topk_groups, float routed_scaling,
                          int renormalize, int ld, int* status, cudaStream_t s) {
  if (rows <= 0 || E <= 0 || E > ROUTE_MAX_E || top_k < 1 || top_k > 32 || top_k > E) return FF_HOST_BAD_SHAPE;
  if (n_groups < 1 || n_groups > 32 || E % n_groups || topk_groups < 1 || topk_groups > n_groups) return FF_HOST_BAD_SHAPE;
  moe_topk_kernel<<<(rows + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, 0, s>>>(
      (const __nv_bfloat16*)logits, bias, out_w, out_ids, rows, E, top_k, score_mode, n_groups, topk_groups,
      routed_scaling, renormalize, ld, status);
  return launch_result();
}

// counts/cursors: int32[E_local]; seg_off: int32[E_local + 1]; pos: int32[rows * top_k];
// sorted: bf16 [capacity, hidden]. Experts [e_lo, e_hi) are local.
FF_EXPORT int ff_moe_dispatch_local(const void* x, const int* ids, int rows, int top_k, int hidden, int ldx, int E,
                                    int e_lo, int e_hi, int* counts, int* seg_off, int* cursors, void* sorted,
                                    int* pos, int capacity, int* status, cudaStream_t s) {
  const int el = e_hi - e_lo;
  if (rows <= 0 || top_k < 1 || hidden % 8 || el < 1 || el > 1024 || ldx % 8) return FF_HOST_BAD_SHAPE;
  cudaError_t e = cudaMemsetAsync(counts, 0, (size_t)el * 4, s);
  if (e != cudaSuccess) return (int)e;
  const int n = rows * top_k;
  moe_count_kernel<<<(n + 255) / 256, 256, 0, s>>>(ids, n, E, e_lo, e_hi, counts, status);
  moe_scan_kernel<<<1, 1024, 0, s>>>(counts, seg_off, cursors, el, capacity, status);
  moe_permute_kernel<<<n, 128, 0, s>>>((const __nv_bfloat16*)x, ids, seg_off, cursors, (__nv_bfloat16*)sorted, pos,
                                       hidden, top_k, e_lo, e_hi, capacity, ldx);
  return launch_result();
}

FF_EXPORT int ff_moe_grouped_gemm(const void* xs, const void* w, void* y, const int* seg_off, const int* counts,
                                  int E_local, int Nw, int K, int capacity, int ldy, int epi, int* status,
                                  cudaStream_t s) {
  if (E_local < 1 || Nw % 128 || K % 8 || capacity % 16) return FF_HOST_BAD_SHAPE;
  if (epi == 1 && ldy < Nw / 2) return FF_HOST_BAD_SHAPE;
  if (ldy % 8) return FF_HOST_BAD_ALIGN;
  CUtensorMap tmW, tmX;
  int r = make_tmap_2d(&tmW, w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, (uint64_t)E_local * Nw, (uint64_t)K * 2, GBK, GBM);
  if (r) return r;
  r = make_tmap_2d(&tmX, xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, K, capacity, (uint64_t)K * 2, GBK, 16);
  if (r) return r;
  const int staging = 64 * GBM * 4;                      // 32 KiB
  // decode-sized calls (on average at most 24 padded rows per expert): an expert tile is short, so half the pipeline
  // memory per CTA lets two CTAs share an SM and one streams while the other sets up or drains (FF_MOE_SMALL=0: off)
  static const int small_on = [] { const char* ev = getenv("FF_MOE_SMALL"); return (ev && ev[0] == '0') ? 0 : 1; }();
  const bool small = small_on && (long long)capacity <= 24ll * E_local;
  const int pipe_bytes = small ? 76 * 1024 : 3 * (GBM * GBK * 2 + G_TOK * GBK * 2);   // 3 full-width stages = 144 KiB
  const int smem = staging + pipe_bytes + 1024;
  r = opt_in_smem(moe_grouped_gemm_kernel, 200 * 1024); if (r) return r;
  dim3 grid(Nw / GBM, E_local);
  moe_grouped_gemm_kernel<<<grid, 192, smem, s>>>(tmW, tmX, (__nv_bfloat16*)y, seg_off, counts, Nw, K, ldy, epi,
                                                  pipe_bytes, staging, status, capacity);
  return launch_result();
}

FF_EXPORT int ff_moe_combine(const void* y, const int* pos, const int* ids, const float* w, void* out, int rows,
                             int hidden, int top_k, int ldy, int accumulate, cudaStream_t s) {
  if (rows <= 0 || hidden % 8 || top_k < 1 || top_k > 16 || ldy % 8) return FF_HOST_BAD_SHAPE;
  moe_combine_kernel<<<rows, 256, 0, s>>>((const __nv_bfloat16*)y, pos, ids, w, (__nv_bfloat16*)out, hidden, top_k,
                                          ldy, accumulate);
  return launch_result();
}
