// Host-side tensor-map encoding.  The driver entry point is resolved at run time through the
// CUDA runtime so that the library links against cudart only and loads on a machine without
// a driver (where every compute entry point then fails with ZEN_ERR_DRIVER / ZEN_ERR_LAUNCH).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <utility>
#include <mutex>
#include <set>
#include "../../include/zenith_b200.h"
#include "zen_common.cuh"

namespace zen {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Rank-`rank` tiled map with 128-byte swizzle; dims/strides innermost first, strides in bytes
// for dims 1..rank-1.  Out-of-bounds elements read as zero.
inline int encode_tmap(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box,
                       CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return ZEN_ERR_DRIVER;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) {
      if (strides_bytes[i - 1] % 16) return ZEN_ERR_UNSUPPORTED;
      gstr[i - 1] = strides_bytes[i - 1];
    }
  }
  if (reinterpret_cast<uintptr_t>(base) % 16) return ZEN_ERR_UNSUPPORTED;
  CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ZEN_OK : ZEN_ERR_DRIVER;
}

inline int encode_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                          uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                          CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  const uint64_t dims[2] = {inner, outer};
  const uint64_t str[1] = {row_stride_bytes};
  const uint32_t box[2] = {box_inner, box_outer};
  return encode_tmap(map, dt, 2, base, dims, str, box, swizzle);
}

// Launch with the programmatic-stream-serialization attribute (see grid_dependency_wait()).  Only for
// kernels that execute grid_dependency_wait() before touching global data.  `family` is tested against
// ZEN_PDL_FAMILIES, a build-time constant (1 = GEMM, 2 = attention, 4 = row kernels; default: GEMM only).
// Early launch pays off for the GEMMs (long set-up, one CTA per SM); for the short row kernels the
// early-resident CTAs only got in the way (measured: 7.1 vs 5.9 us per LayerNorm).
// (the constant and the family bits live in zen_common.cuh, where the kernels see them too)
constexpr int pdl_mask() { return ZEN_PDL_FAMILIES; }

template <typename... KArgs, typename... Args>
inline int launch_pdl(int family, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl_mask() & family) ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  return ZEN_OK;
}

// Opt a kernel in to more than 48 KB of dynamic shared memory, once per (kernel, device).
inline int ensure_dynamic_smem(const void* kernel, size_t smem) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, dev})) return ZEN_OK;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) {
    cudaGetLastError();
    return ZEN_ERR_LAUNCH;
  }
  done.insert({kernel, dev});
  return ZEN_OK;
}

inline int num_sms() {
  static int cached[64] = {};
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  cached[dev] = v;
  return v;
}

}  // namespace zen
