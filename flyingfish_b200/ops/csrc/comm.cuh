// Peer-memory communication primitives shared by the fused compute+collective kernels.
//
// Every rank owns one "arena" of symmetric memory (same layout on every rank, mapped into every
// peer's address space through NVLink). Layout, in bytes from the arena base:
//
//   [0, 64)                      control: int32 epoch, int32 done counter (local use only)
//   [FLAG_OFF, +world*MAX_FLAGS*4)   arrival flags, indexed [source rank][slot]
//   [DATA_OFF, ...)              two parity halves of `half_bytes`, each holding `world` slots
//                                of `slot_bytes` (one per source rank)
//
// Protocol of one collective launch (identical launch sequence on every rank):
//   epoch = control.epoch + 1 (read once per CTA at kernel start; the last CTA to finish stores
//   it back), parity = epoch & 1. A producer pushes its data into slot[parity][my_rank] of each
//   peer with plain stores, fences at system scope and then release-stores `epoch` into
//   flag[my_rank][slot] of that peer. A consumer acquire-polls its LOCAL flags (bounded by a
//   timer; on time-out it records FF_ERR_TIMEOUT and gives up) and then reads only local memory.
//   Because every launch ends with all ranks having exchanged flags, data written in launch i
//   cannot be overwritten before launch i+2, which is why two parity halves are enough.
//
// No TMA multicast and no library kernel ever touches peer memory; all peer traffic is plain
// st.global / ld.global (or multimem on an NVLS mapping) issued by these kernels.
#pragma once
#include "ptx.cuh"

namespace ff {

constexpr int MAX_RANKS = 8;
constexpr int MAX_FLAGS = 4096;
constexpr int CTRL_BYTES = 256;
constexpr int FLAG_OFF = CTRL_BYTES;
constexpr int DATA_OFF = FLAG_OFF + MAX_RANKS * MAX_FLAGS * 4;   // 131328, 256-byte aligned

struct PeerArena {
  uint8_t* base[MAX_RANKS];     // arena base of every rank as mapped in this process
  int rank;
  int world;
  long long half_bytes;         // bytes of one parity half of the data area
  long long slot_bytes;         // bytes of one source-rank slot inside a half
  uint8_t* mc_base;             // NVLS multicast mapping of the same arena (null: plain peer stores only)
  int mc_oneshot;               // with mc_base: every rank multicasts its partial to all ranks (one flag round) and sums locally
};

__device__ __forceinline__ int* arena_epoch(const PeerArena& a) { return reinterpret_cast<int*>(a.base[a.rank]); }
__device__ __forceinline__ int* arena_done(const PeerArena& a) { return reinterpret_cast<int*>(a.base[a.rank]) + 1; }
__device__ __forceinline__ int* arena_flag(const PeerArena& a, int on_rank, int src_rank, int slot) {
  return reinterpret_cast<int*>(a.base[on_rank] + FLAG_OFF) + src_rank * MAX_FLAGS + slot;
}
__device__ __forceinline__ uint8_t* arena_slot(const PeerArena& a, int on_rank, int parity, int src_rank) {
  return a.base[on_rank] + DATA_OFF + (long long)parity * a.half_bytes + (long long)src_rank * a.slot_bytes;
}

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v; asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ int ld_volatile(const int* p) {
  int v; asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}

// ---- NVLS (multimem) accessors: one instruction acts on the same arena offset of every rank ------------
// multicast address of a location given by its address in this rank's own mapping
template <typename T>
__device__ __forceinline__ T* arena_mc(const PeerArena& a, T* local) {
  return reinterpret_cast<T*>(a.mc_base + (reinterpret_cast<uint8_t*>(local) - a.base[a.rank]));
}
// sum over all ranks of eight BF16 values, accumulated in FP32 inside the switch
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// store eight BF16 values to every rank
__device__ __forceinline__ void multimem_st_bf16x8(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// release-store of a flag word to every rank
__device__ __forceinline__ void multimem_st_release(int* mc, int v) {
  asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

// Bounded wait until *flag has reached `epoch` (wrap-safe comparison).
__device__ __forceinline__ bool wait_flag(const int* flag, int epoch, int* status, int kid, int where) {
  if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((++it & 63u) == 0 && globaltimer_ns() - t0 > FF_WAIT_NS) {
      set_status(status, kid, FF_ERR_TIMEOUT, where, epoch);
      return false;
    }
  }
}

// Called by every CTA when it is done with the arena; the last one publishes the new epoch.
__device__ __forceinline__ void arena_finish(const PeerArena& a, int epoch, int total_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(arena_done(a), 1);
    if (prev == total_ctas - 1) {
      *arena_done(a) = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(arena_epoch(a)) = epoch;
    }
  }
}

}  // namespace ff
