// Collective kernels over peer memory (NVLink 5 / NVSwitch), see comm.cuh for the protocol.
//   allreduce_oneshot : every rank pushes its vector into each peer's slot, flags, then sums the
//                       `world` slots in rank order (bitwise identical result on every rank).
//                       Optional fused residual-add + RMSNorm on the reduced rows.
//   allgather_push    : every rank pushes its shard into slot[rank] of each peer and the result is
//                       read locally (used for vocab-parallel argmax candidates and small AGs).
//   transport self-test kernels: pattern fill / verify, used at start-up to check the mapping of
//                       every peer (the reference verifies its transport with a byte pattern and
//                       a planted flip, src/backend/cuda/mod.rs:487-664).
#include "comm.cuh"
#include "host_util.h"

namespace ff {

// x: bf16 [numel]; out: bf16 [numel]. numel % 8 == 0. grid <= MAX_FLAGS CTAs, each owns a
// contiguous chunk. If `norm_w` is given the vector is [rows][hidden] and every CTA owns whole
// rows: out_res = res + sum (rounded to bf16), out = rmsnorm(out_res) * w.
__global__ void __launch_bounds__(512)
allreduce_oneshot_kernel(PeerArena a, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                         long long numel, int chunk_vecs, int* status) {
  const int epoch = ld_volatile(arena_epoch(a)) + 1;
  const int parity = epoch & 1;
  const long long nvec = numel >> 3;
  const long long v0 = (long long)blockIdx.x * chunk_vecs;
  const long long v1 = min(nvec, v0 + chunk_vecs);
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  // push my chunk to every peer
  for (int pi = 1; pi < a.world; ++pi) {
    const int p = (a.rank + pi) % a.world;
    uint4* dst = reinterpret_cast<uint4*>(arena_slot(a, p, parity, a.rank));
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) dst[v] = xv[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int pi = 1; pi < a.world; ++pi) {
      const int p = (a.rank + pi) % a.world;
      st_release_sys(arena_flag(a, p, a.rank, blockIdx.x), epoch);
    }
  }
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < a.world && threadIdx.x != a.rank) {
    if (!wait_flag(arena_flag(a, a.rank, threadIdx.x, blockIdx.x), epoch, status, KID_AR, threadIdx.x)) ok_s = 0;
  }
  __syncthreads();
  if (ok_s) {
    for (long long v = v0 + threadIdx.x; v < v1; v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int r = 0; r < a.world; ++r) {
        const uint4 d = (r == a.rank) ? xv[v] : reinterpret_cast<const uint4*>(arena_slot(a, a.rank, parity, r))[v];
        const uint32_t* dp = reinterpret_cast<const uint32_t*>(&d);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = unpack_bf16x2(dp[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out)[v] = o;
    }
  }
  arena_finish(a, epoch, gridDim.x);
}

// Generic small all-gather: every rank contributes `bytes` (multiple of 16); out receives
// world * bytes in rank order. One CTA.
__global__ void __launch_bounds__(256)
allgather_push_kernel(PeerArena a, const uint8_t* __restrict__ x, uint8_t* __restrict__ out, int bytes, int* status) {
  const int epoch = ld_volatile(arena_epoch(a)) + 1;
  const int parity = epoch & 1;
  const int nvec = bytes >> 4;
  for (int pi = 1; pi < a.world; ++pi) {
    const int p = (a.rank + pi) % a.world;
    uint4* dst = reinterpret_cast<uint4*>(arena_slot(a, p, parity, a.rank));
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = reinterpret_cast<const uint4*>(x)[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int pi = 1; pi < a.world; ++pi) st_release_sys(arena_flag(a, (a.rank + pi) % a.world, a.rank, 0), epoch);
  }
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < a.world && threadIdx.x != a.rank)
    if (!wait_flag(arena_flag(a, a.rank, threadIdx.x, 0), epoch, status, KID_AR, 100 + threadIdx.x)) ok_s = 0;
  __syncthreads();
  if (ok_s) {
    for (int r = 0; r < a.world; ++r) {
      const uint4* src = (r == a.rank) ? reinterpret_cast<const uint4*>(x)
                                       : reinterpret_cast<const uint4*>(arena_slot(a, a.rank, parity, r));
      uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * bytes);
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = src[v];
    }
  }
  arena_finish(a, epoch, 1);
}

// start-up self test: write pattern(rank, i) into slot[0][rank] of every peer
__global__ void transport_fill_kernel(PeerArena a, int words, unsigned salt) {
  for (int pi = 0; pi < a.world; ++pi) {
    const int p = (a.rank + pi) % a.world;
    unsigned* dst = reinterpret_cast<unsigned*>(arena_slot(a, p, 0, a.rank));
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += gridDim.x * blockDim.x)
      dst[i] = (unsigned)(a.rank * 0x9E3779B9u) ^ (unsigned)(i * 2654435761u) ^ salt;
  }
}
// count mismatches of what every source rank wrote into my slots
__global__ void transport_verify_kernel(PeerArena a, int words, unsigned salt, int* mismatches) {
  int bad = 0;
  for (int r = 0; r < a.world; ++r) {
    const unsigned* src = reinterpret_cast<const unsigned*>(arena_slot(a, a.rank, 0, r));
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < words; i += gridDim.x * blockDim.x)
      if (src[i] != ((unsigned)(r * 0x9E3779B9u) ^ (unsigned)(i * 2654435761u) ^ salt)) ++bad;
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace ff
using namespace ff;

static int fill_arena(PeerArena& a, const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                      long long slot_bytes) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return FF_HOST_BAD_SHAPE;
  if (slot_bytes % 256 || half_bytes < slot_bytes * world) return FF_HOST_BAD_ALIGN;
  for (int i = 0; i < MAX_RANKS; ++i) a.base[i] = i < world ? reinterpret_cast<uint8_t*>(ptrs[i]) : nullptr;
  a.rank = rank; a.world = world; a.half_bytes = half_bytes; a.slot_bytes = slot_bytes;
  return 0;
}

FF_EXPORT long long ff_arena_data_offset() { return DATA_OFF; }
FF_EXPORT int ff_arena_max_flags() { return MAX_FLAGS; }

FF_EXPORT int ff_allreduce_oneshot(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                                   long long slot_bytes, const void* x, void* out, long long numel, int* status,
                                   cudaStream_t s) {
  PeerArena a = {};
  if (int r = fill_arena(a, ptrs, rank, world, half_bytes, slot_bytes)) return r;
  if (numel <= 0 || numel % 8 || numel * 2 > slot_bytes) return FF_HOST_TOO_LARGE;
  const long long nvec = numel / 8;
  // chunks of >= 512 vectors (8 KiB) so a CTA's flag traffic is amortised; at most 128 CTAs
  int ctas = (int)((nvec + 511) / 512);
  if (ctas > 128) ctas = 128;
  if (ctas < 1) ctas = 1;
  const int chunk = (int)((nvec + ctas - 1) / ctas);
  ctas = (int)((nvec + chunk - 1) / chunk);
  allreduce_oneshot_kernel<<<ctas, 512, 0, s>>>(a, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, numel, chunk, status);
  return launch_result();
}

FF_EXPORT int ff_allgather_push(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                                long long slot_bytes, const void* x, void* out, int bytes, int* status, cudaStream_t s) {
  PeerArena a = {};
  if (int r = fill_arena(a, ptrs, rank, world, half_bytes, slot_bytes)) return r;
  if (bytes <= 0 || bytes % 16 || bytes > slot_bytes) return FF_HOST_TOO_LARGE;
  allgather_push_kernel<<<1, 256, 0, s>>>(a, (const uint8_t*)x, (uint8_t*)out, bytes, status);
  return launch_result();
}

FF_EXPORT int ff_transport_fill(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                                long long slot_bytes, int words, unsigned salt, cudaStream_t s) {
  PeerArena a = {};
  if (int r = fill_arena(a, ptrs, rank, world, half_bytes, slot_bytes)) return r;
  if ((long long)words * 4 > slot_bytes) return FF_HOST_TOO_LARGE;
  transport_fill_kernel<<<32, 256, 0, s>>>(a, words, salt);
  return launch_result();
}

FF_EXPORT int ff_transport_verify(const unsigned long long* ptrs, int rank, int world, long long half_bytes,
                                  long long slot_bytes, int words, unsigned salt, int* mismatches, cudaStream_t s) {
  PeerArena a = {};
  if (int r = fill_arena(a, ptrs, rank, world, half_bytes, slot_bytes)) return r;
  transport_verify_kernel<<<32, 256, 0, s>>>(a, words, salt, mismatches);
  return launch_result();
}
