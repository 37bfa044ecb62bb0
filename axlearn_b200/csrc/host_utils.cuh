// Host-side helpers shared by the launchers: TMA descriptor encoding (driver entry point
// resolved through the runtime, so the library does not link against libcuda), device
// properties, and the global status word that kernels use to report bounded-wait timeouts.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace axb {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        p == nullptr) {
      fprintf(stderr, "axb: cannot resolve cuTensorMapEncodeTiled\n");
      return nullptr;
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Encodes a tiled map of `rank` dims (innermost first). strides_bytes has rank-1 entries
// (stride of dim 1.. in bytes; each a multiple of 16). Returns 0 on success.
inline int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                           const uint64_t* dims, const uint64_t* strides_bytes,
                           const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -1;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t bdims[5];
  cuuint32_t estrides[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    bdims[i] = box[i];
    estrides[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(map, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims,
                  gstrides, bdims, estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "axb: cuTensorMapEncodeTiled failed (%d): rank %d dims", static_cast<int>(r),
            rank);
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %llu", (unsigned long long)dims[i]);
    fprintf(stderr, " box");
    for (int i = 0; i < rank; ++i) fprintf(stderr, " %u", box[i]);
    fprintf(stderr, " base %p\n", base);
    return -2;
  }
  return 0;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace axb
