// Warp-level mma.sync m16n8k16 (BF16 x BF16 -> FP32) and ldmatrix helpers for small attention tiles whose operands are
// produced in shared memory by the CTA itself (de-quantised cache rows), where a tcgen05 pipeline has nothing to stream.
#pragma once
#include <cstdint>

namespace ff {

__device__ __forceinline__ void ms_ldsm4(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ms_ldsm4t(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ms_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// byte offset of 16-byte chunk c of row r in a [rows][chunks * 8] bf16 tile whose chunk index is XORed with r % 8
__device__ __forceinline__ uint32_t ms_off(int r, int c, int chunks) { return (uint32_t)((r * chunks + ((c & ~7) | ((c ^ r) & 7))) * 16); }

}  // namespace ff
