// Host-side helpers shared by the launchers: TMA tensor-map encoding through the driver
// entry point (no link-time dependency on libcuda), launch error mapping, device queries.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <map>
#include <mutex>
#include <utility>

namespace ff {

// Launcher return codes (negative = host-side refusal, positive = cudaError_t).
enum HostErr : int {
  FF_HOST_OK = 0,
  FF_HOST_BAD_SHAPE = -1,
  FF_HOST_BAD_ALIGN = -2,
  FF_HOST_NO_DRIVER = -3,
  FF_HOST_TMAP_FAIL = -4,
  FF_HOST_TOO_LARGE = -5,
  FF_HOST_UNSUPPORTED = -6,
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// 2-D row-major tensor [outer, inner] with `row_bytes` pitch; box [box_outer, box_inner];
// 128-byte swizzle when the box's inner extent is exactly 128 bytes, none otherwise.
inline int make_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                        uint64_t inner, uint64_t outer, uint64_t row_bytes, uint32_t box_inner,
                        uint32_t box_outer, bool swizzle128 = true) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return FF_HOST_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_bytes & 15)) return FF_HOST_BAD_ALIGN;
  if (box_inner * elem_bytes > 128 && swizzle128) return FF_HOST_BAD_SHAPE;
  if (box_outer > 256 || box_inner > 256) return FF_HOST_BAD_SHAPE;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FF_HOST_OK : FF_HOST_TMAP_FAIL;
}

// 3-D tensor [d2, d1, d0] (d0 innermost) with byte strides for d1 and d2.
inline int make_tmap_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                        uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes,
                        uint32_t b0, uint32_t b1, uint32_t b2, bool swizzle128 = true) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return FF_HOST_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (stride1_bytes & 15) || (stride2_bytes & 15)) return FF_HOST_BAD_ALIGN;
  if (b0 * elem_bytes > 128 && swizzle128) return FF_HOST_BAD_SHAPE;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FF_HOST_OK : FF_HOST_TMAP_FAIL;
}

constexpr int FF_MAX_DEVICES = 64;

// index of the current device, clamped into the per-device caches below
inline int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  return dev < 0 ? 0 : (dev >= FF_MAX_DEVICES ? FF_MAX_DEVICES - 1 : dev);
}

// SM count of the current device (cached per device: one process may drive several GPUs)
inline int sm_count() {
  static int n[FF_MAX_DEVICES] = {};
  const int dev = current_device();
  if (n[dev] == 0) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

inline int launch_result() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FF_HOST_OK : static_cast<int>(e);
}

// Programmatic dependent launch. A kernel started through launch_pdl may begin while the previous
// kernel of the stream is still running (its prologue, and loads of data that no kernel writes,
// overlap that kernel's tail); every such kernel executes griddepcontrol.wait before it touches
// memory a predecessor produces, and griddepcontrol.launch_dependents early so that its own
// successor may do the same. FLYINGFISH_PDL=0 turns the attribute off (plain stream order).
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("FLYINGFISH_PDL"); v = (e != nullptr && e[0] == '0') ? 0 : 1; }
  return v != 0;
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute at[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = (unsigned)cluster; at[n].val.clusterDim.y = 1; at[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = at; cfg.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  return FF_HOST_OK;
}

// Opt a kernel in to `bytes` of dynamic shared memory on the CURRENT device. The attribute is per
// device, so the "already done" record is keyed by (device, kernel); launchers call this before
// every launch and pay a map look-up when nothing is to be done. Safe from several host threads.
template <typename K>
inline int opt_in_smem(K kernel, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> done;
  const std::pair<int, const void*> key(current_device(), reinterpret_cast<const void*>(kernel));
  std::lock_guard<std::mutex> lock(mu);
  auto it = done.find(key);
  if (it != done.end() && it->second >= bytes) return FF_HOST_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) { cudaGetLastError(); return static_cast<int>(e); }
  done[key] = bytes;
  return FF_HOST_OK;
}

}  // namespace ff

#define FF_EXPORT extern "C" __attribute__((visibility("default")))
