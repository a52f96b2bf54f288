// Blackwell (sm_100a) PTX building blocks shared by every kernel in this library:
// mbarrier with bounded waits, TMA bulk-tensor loads, tcgen05 MMA / TMEM management,
// UMMA shared-memory and instruction descriptors, and the device status word.
//
// Error policy: nothing here traps or spins without a limit. A wait that does not
// complete within FF_WAIT_NS nanoseconds records (kernel id, code, detail) in the status
// word and returns false; the caller unwinds (frees TMEM, leaves the kernel).
// The reference engine traps on contract violations (kernels/gpu_compat.cuh FF_TRAP);
// this library reports through memory instead so a shared GPU context stays usable.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda.h>
#include <stdint.h>

namespace ff {

// ---------------------------------------------------------------------------------------
// Status word: int32[4] in global memory = {code, kernel_id, detail0, detail1}.
// First error wins. Host reads it at its existing sync points.
// ---------------------------------------------------------------------------------------
enum StatusCode : int {
  FF_OK = 0,
  FF_ERR_TIMEOUT = 1,      // a bounded wait ran out
  FF_ERR_CONTRACT = 2,     // shape / index contract violated by metadata
  FF_ERR_BOUNDS = 3,       // index outside a table (bad token id, bad block id ...)
  FF_ERR_NONFINITE = 4,    // non-finite value seen by a sticky scan
  FF_ERR_CAPACITY = 5,     // a device-side buffer would overflow
  FF_ERR_DOUBLE_WRITE = 6, // debug build: an element with a single-writer contract was written twice in one launch
};

enum KernelId : int {
  KID_GEMM_BF16 = 1, KID_GEMM_SKINNY = 2, KID_EMBED = 3, KID_NORM = 4, KID_ROPE_KV = 5,
  KID_ACT = 6, KID_ATTN_DECODE = 7, KID_ATTN_PREFILL = 8, KID_SAMPLE = 9, KID_AR = 10,
  KID_GEMM_AR = 11, KID_AG_GEMM = 12, KID_GEMM_RS = 13, KID_MOE_ROUTE = 14,
  KID_MOE_DISPATCH = 15, KID_MOE_GEMM = 16, KID_MOE_COMBINE = 17, KID_QUANT = 18,
  KID_GEMM_FP8 = 19, KID_GEMM_NVFP4 = 20, KID_MLA = 21, KID_VERIFY = 22, KID_KV = 23,
  KID_DSA = 24, KID_LATENT = 25, KID_GDN = 26, KID_MHC = 27, KID_MARKOV = 28, KID_VISION = 29,
  KID_CHAIN = 30,
};

__device__ __forceinline__ void set_status(int* status, int kid, int code, int d0 = 0, int d1 = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = kid; status[2] = d0; status[3] = d1;
    __threadfence_system();
  }
}

// ---------------------------------------------------------------------------------------
// Debug build (-DFF_DEBUG_CHECKS): single-writer ledger. Scratch with the contract "every element is written by
// exactly one block per launch" (split-K partial rows, attention split partials, the KV-cache rows of a step) claims
// its element here; a second claim in the same launch epoch sets FF_ERR_DOUBLE_WRITE with (region, index). The host
// enlarges the status buffer: word 9 = epoch (bumped before every launch), word 10 = entries per region, word 11 =
// claims that fell outside a region (not checked), ledger from word 16 on, DBG_REGIONS regions. Compiled out otherwise.
// ---------------------------------------------------------------------------------------
enum DbgRegion : int { DBG_GEMM_PARTIAL = 0, DBG_ATTN_PARTIAL = 1, DBG_KV_K = 2, DBG_KV_V = 3, DBG_REGIONS = 4 };
#ifdef FF_DEBUG_CHECKS
__device__ __forceinline__ void dbg_write_once(int* status, int kid, int region, long long index) {
  if (status == nullptr) return;
  const int len = status[10], epoch = status[9];
  if (len <= 0 || index < 0 || index >= len || region < 0 || region >= DBG_REGIONS) { atomicAdd(&status[11], 1); return; }
  const int prev = atomicExch(&status[16 + (size_t)region * len + index], epoch);
  if (prev == epoch) set_status(status, kid, FF_ERR_DOUBLE_WRITE, region, (int)index);
}
#define FF_DBG_CHECK(cond, status, kid, d0, d1) do { if (!(cond)) set_status((status), (kid), FF_ERR_BOUNDS, (d0), (d1)); } while (0)
#else
__device__ __forceinline__ void dbg_write_once(int*, int, int, long long) {}
#define FF_DBG_CHECK(cond, status, kid, d0, d1) do {} while (0)
#endif

#ifndef FF_WAIT_NS
#define FF_WAIT_NS 2000000000ull   // 2 s: far above any legitimate wait in this library
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}

// ---------------------------------------------------------------------------------------
// Device timeline (compiled in only with -DFF_TIMELINE; the tracing build of the library).
// The status buffer is then larger: int32 word 8 counts records, 16-byte records start at word 16:
// {globaltimer lo, hi, kernel id << 16 | phase, SM id << 20 | linear block index}. One thread per CTA
// calls FF_TL at the points of interest; the host reads the buffer after a synchronise.
// ---------------------------------------------------------------------------------------
#ifdef FF_TIMELINE
#ifndef FF_TL_CAP
#define FF_TL_CAP (1 << 18)
#endif
__device__ __forceinline__ void timeline_record(int* status, int kid, int phase) {
  if (status == nullptr) return;
  const int i = atomicAdd(status + 8, 1);
  if (i >= FF_TL_CAP) return;
  const uint64_t t = globaltimer_ns();
  uint32_t sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
  int4 rec;
  rec.x = (int)(uint32_t)t; rec.y = (int)(uint32_t)(t >> 32);
  const uint32_t lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  rec.z = (kid << 16) | (phase & 0xffff); rec.w = (int)((sm << 20) | (lin & 0xfffffu));
  reinterpret_cast<int4*>(status + 16)[i] = rec;
}
#define FF_TL(status, kid, phase) timeline_record(status, kid, phase)
#else
#define FF_TL(status, kid, phase) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t.reg .b32 R;\n\t"
      "elect.sync R|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred;
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait. `abort_flag` (shared memory) lets the first role that gives up release the
// others quickly instead of each running out its own limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int kid, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++it & 255u) == 0) {
      if (abort_flag && *abort_flag) return false;
      if (globaltimer_ns() - t0 > FF_WAIT_NS) {
        if (abort_flag) *abort_flag = 1;
        set_status(status, kid, FF_ERR_TIMEOUT, where, (int)parity);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), loads only, never with cluster multicast.
// The innermost coordinate times the element size must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// L2 policy for data that is read once (weight streams): evict it before anything else
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// ---- thread-block clusters: barrier over all threads of the cluster, distributed shared memory --
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {     // every thread of every CTA, warps converged
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// split form: arrive early (e.g. at kernel entry), wait where the peers' progress is needed
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank)); return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

__device__ __forceinline__ void st_dsmem_f4(uint32_t addr, float4 v) {
  asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// wait: everything the preceding kernel in the stream wrote is visible after this returns (no-op
// when the kernel was launched without the programmatic-serialisation attribute).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// trigger: the next kernel in the stream may start its prologue now
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
// Untiled bulk copy shared -> global (16-byte aligned both sides, size a multiple of 16). The destination may be a
// peer GPU's memory: the copy engine keeps many write requests in flight where a warp's own stores would not.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gmem_dst)), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, UMMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// tcgen05 / TMEM
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {        // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc]; one thread issues.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// A operand read from TMEM (D = A[tmem] * B[smem]).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// FP8/FP6/FP4 operand kinds (E4M3 etc.), FP32 accumulate.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// mbarrier arrives once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// TMEM -> registers: 32 lanes x 32 bit, N consecutive columns; warp w of a warpgroup may only
// touch lanes [32*(w%4), 32*(w%4)+32).
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// registers -> TMEM (same lane restriction as loads)
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle (matches CU_TENSOR_MAP_SWIZZLE_128B).
//  K-major operand : rows of 128 bytes (64 bf16 / 128 fp8), 8-row groups 1024 B apart (SBO);
//                    LBO unused.
//  MN-major operand: 128 bytes contiguous along M/N, 8 K-rows per 1024-B atom; LBO = byte step
//                    between 64-element MN blocks, SBO = byte step between 8-row K groups.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}
// Instruction descriptor for kind::f16 / kind::f8f6f4 with FP32 accumulation.
//  fmt: kind::f16 -> 0 = F16, 1 = BF16 ; kind::f8f6f4 -> 0 = E4M3, 1 = E5M2, 5 = E2M1
//  major: 0 = K-major, 1 = MN-major
__host__ __device__ constexpr uint32_t umma_idesc(int a_fmt, int b_fmt, int a_major, int b_major, int m, int n) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)a_major << 15) |
         ((uint32_t)b_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---------------------------------------------------------------------------------------
// small numeric helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace ff
