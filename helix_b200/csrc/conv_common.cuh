// Pieces shared by the convolution kernels that keep their input resident in shared memory (conv_f16_halo.cu,
// conv_f16_stem.cu, conv_f16_rows.cu).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace helix {

// cuTensorMapEncodeTiled, looked up once through the runtime (no link against libcuda); null when unavailable.
// Defined in conv_f16_halo.cu.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn conv_tensor_map_encoder();

// 4-D tiled load (C, W, H, N); coordinates may be negative or beyond the tensor: those elements
// arrive as zeros.  c * 2 bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* desc, uint64_t* bar, int c, int w, int h,
                                            int n) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n)
      : "memory");
}

// two fp32 values rounded to nearest-even fp16, packed low / high
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

}  // namespace helix
