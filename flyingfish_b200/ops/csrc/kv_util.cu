// Paged KV-cache row utilities: move the K/V rows of chosen cache slots to other slots in every layer at once.
// Speculative tree verification writes the rows of all tree nodes behind the committed prefix; after acceptance
// the rows of the accepted path are compacted onto consecutive positions. Two launches for the whole model
// (gather into a staging buffer, scatter out of it: overlapping source and destination sets are safe), instead of
// an indexing operation per layer and per tensor. Counterpart of the reference's tree_kv_gather / tree_kv_scatter
// (kernels/tree/meta.cu), for a block cache laid out [blocks, kv heads, block size, head dim].
#include "ptx.cuh"
#include "host_util.h"

namespace ff {

// caches: device array of base pointers (one per tensor: K and V of every layer that has them); slot = block *
// block_size + offset. Row of tensor c for slot s and head h: caches[c] + ((block * heads + h) * block_size + off) * dim.
// grid (moves, tensors), threads cover heads * dim / 8 vectors of 16 bytes.
template <bool GATHER>
__global__ void kv_move_rows_kernel(const unsigned long long* __restrict__ caches, const int* __restrict__ slots,
                                    uint4* __restrict__ staging, int heads, int block_size, int dim, int num_blocks,
                                    int* status) {
  pdl_trigger();
  pdl_wait();
  const int m = blockIdx.x, c = blockIdx.y;
  const int slot = slots[m];
  const int blk = slot / block_size, off = slot - blk * block_size;
  if (slot < 0 || blk >= num_blocks) { if (threadIdx.x == 0) set_status(status, KID_KV, FF_ERR_BOUNDS, m, slot); return; }
  const int vec_per_head = dim / 8;
  const int nvec = heads * vec_per_head;
  uint4* base = reinterpret_cast<uint4*>(caches[c]);
  uint4* stage = staging + ((size_t)c * gridDim.x + m) * nvec;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const int h = i / vec_per_head, v = i - h * vec_per_head;
    uint4* row = base + (((size_t)blk * heads + h) * block_size + off) * vec_per_head + v;
    if (GATHER) stage[i] = *row; else *row = stage[i];
  }
}

}  // namespace ff
using namespace ff;

// staging: at least moves * tensors * heads * dim * 2 bytes. src_slots / dst_slots: device int32[moves].
FF_EXPORT int ff_kv_move_rows(const unsigned long long* caches, int tensors, const int* src_slots, const int* dst_slots,
                              int moves, void* staging, int heads, int block_size, int dim, int num_blocks, int* status,
                              cudaStream_t s) {
  if (moves <= 0 || tensors <= 0 || heads <= 0 || dim % 8 || block_size <= 0) return FF_HOST_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(staging) & 15) return FF_HOST_BAD_ALIGN;
  dim3 grid(moves, tensors);
  const int threads = heads * dim / 8 >= 256 ? 256 : 64;
  if (int r = launch_pdl(kv_move_rows_kernel<true>, grid, dim3(threads), 0, s, 0, caches, src_slots,
                         static_cast<uint4*>(staging), heads, block_size, dim, num_blocks, status)) return r;
  return launch_pdl(kv_move_rows_kernel<false>, grid, dim3(threads), 0, s, 0, caches, dst_slots,
                    static_cast<uint4*>(staging), heads, block_size, dim, num_blocks, status);
}
