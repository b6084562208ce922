// TMA tensor maps for the operator's [tokens, H, D] tensors: one tiled load (cp.async.bulk.tensor) fetches the
// 64 token rows of one head, either as a plain row-major box or as 64-column boxes in the 128-byte-swizzled
// layout that ldmatrix and tcgen05 operands use.  Rows past the end of the tensor arrive as zeros.
#pragma once

#include <cuda.h>

#include "kda_common.cuh"

namespace kda {

using TmapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library does not link libcuda.
inline TmapEncodeFn tmap_encode_fn() {
  static TmapEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<TmapEncodeFn>(p);
  }();
  return fn;
}

// Map of a [tokens][H][D] tensor with a box of box_cols columns x one head x box_rows tokens.
// Returns 0 on success, nonzero otherwise.
inline int make_rows_tmap(CUtensorMap* m, const void* base, bool fp32, long long tokens, int H, int D, int box_cols, int box_rows,
                          bool swizzle128) {
  TmapEncodeFn fn = tmap_encode_fn();
  if (!fn) return 1;
  const cuuint64_t es = fp32 ? 4 : 2;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(tokens)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * es, static_cast<cuuint64_t>(H) * D * es};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), 1u, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  auto encode = [&] {
    return fn(m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encoder is a driver call and wants a context bound to the calling thread; a host thread that has only been
    // handed work (an autograd worker) may not have one yet.  A runtime call binds the device's primary context.
    cudaFree(nullptr);
    r = encode();
  }
  return r == CUDA_SUCCESS ? 0 : 2;
}

// global -> shared tiled load of the box at (column c0, head c1, token c2); completes `box bytes` on `bar`.
// c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_rows(void* dst_smem, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
               : "memory");
}

}  // namespace kda
