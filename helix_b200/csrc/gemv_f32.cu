// True-fp32 GEMV for 1..8 right-hand sides: Y[i, r] = sum_k W[r, k] * X[i, k], FFMA only.
//
// Counterpart of the reference's mySGemvKernel_Stage4<float> (src_template/Ampere_FP32/
// gemv_template_fp32.cu:153-218), which no reference script builds: W is streamed once with 128-bit
// loads that bypass L1, several loads in flight per thread, each lane of a warp keeps one fused
// multiply-add chain per (row, right-hand side) over the K elements it owns, and the 32 partial sums meet
// in a warp-shuffle tree.  The order of that sum is fixed (lane chains over ascending k, then the xor tree
// 16, 8, 4, 2, 1), so the result is reproducible bit for bit; with split_k > 1 the K slices are summed in
// slice order by a second kernel.
#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace helix {

template <int MRHS, int RPW, int UNROLL>
__global__ void __launch_bounds__(256)
gemv_f32_kernel(const float* __restrict__ W, int64_t ldw, const float* __restrict__ X, int64_t ldx,
                float* __restrict__ Y, int64_t ldy, int64_t ldy_inner, float* __restrict__ partial, int rows, int K,
                int m, int split_k, int k_per_split) {
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int warps_per_block = blockDim.x >> 5;
  const int row_groups = (rows + RPW - 1) / RPW;
  const int ks = blockIdx.y;
  const int k_begin = ks * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);

  for (int g = blockIdx.x * warps_per_block + warp; g < row_groups; g += gridDim.x * warps_per_block) {
    const int r0 = g * RPW;
    float acc[RPW][MRHS];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int i = 0; i < MRHS; ++i) acc[r][i] = 0.0f;
    const float* wrow[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) wrow[r] = W + (int64_t)min(r0 + r, rows - 1) * ldw;

    // a lane owns the four consecutive elements at k0 + 4 * lane of every 128-element stretch
    for (int k0 = k_begin + lane * 4; k0 < k_end; k0 += 128 * UNROLL) {
      uint4 wv[UNROLL][RPW];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = k0 + u * 128;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          if (k < k_end) wv[u][r] = ldg_stream_16(wrow[r] + k);
          else wv[u][r] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = k0 + u * 128;
        if (k < k_end) {
#pragma unroll
          for (int i = 0; i < MRHS; ++i) {
            if (i < m) {
              const float4 xv = __ldg(reinterpret_cast<const float4*>(X + (int64_t)i * ldx + k));
#pragma unroll
              for (int r = 0; r < RPW; ++r) {
                acc[r][i] = fmaf(__uint_as_float(wv[u][r].x), xv.x, acc[r][i]);
                acc[r][i] = fmaf(__uint_as_float(wv[u][r].y), xv.y, acc[r][i]);
                acc[r][i] = fmaf(__uint_as_float(wv[u][r].z), xv.z, acc[r][i]);
                acc[r][i] = fmaf(__uint_as_float(wv[u][r].w), xv.w, acc[r][i]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int i = 0; i < MRHS; ++i) {
        float v = acc[r][i];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        acc[r][i] = v;
      }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (r0 + r < rows) {
#pragma unroll
          for (int i = 0; i < MRHS; ++i) {
            if (i < m) {
              if (split_k == 1) Y[(int64_t)i * ldy + (int64_t)(r0 + r) * ldy_inner] = acc[r][i];
              else partial[((int64_t)ks * m + i) * rows + r0 + r] = acc[r][i];
            }
          }
        }
      }
    }
  }
}

// Sums the split-K partials in slice order (deterministic).
__global__ void gemv_f32_splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ Y, int64_t ldy,
                                              int64_t ldy_inner, int rows, int m, int split_k) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * m) return;
  const int i = idx / rows, r = idx - i * rows;
  float s = 0.0f;
  for (int ks = 0; ks < split_k; ++ks) s += partial[((int64_t)ks * m + i) * rows + r];
  Y[(int64_t)i * ldy + (int64_t)r * ldy_inner] = s;
}

size_t gemv_f32_workspace_bytes(int rows, int m, int split_k) {
  return split_k > 1 ? (size_t)split_k * m * rows * sizeof(float) : 0;
}

int gemv_f32_default_split(int rows, int K, int sm_count) {
  const int groups = (rows + 1) / 2;
  int split = 1;
  // as the fp16 kernel: beyond four warps per SM only very long rows are cut
  while (split < 16 && K / (split * 2) >= 1024 &&
         ((int64_t)groups * split < (int64_t)sm_count * 4 ||
          ((int64_t)groups * split < (int64_t)sm_count * 24 && K / (split * 2) >= 8192)))
    split *= 2;
  return split;
}

template <int MRHS, int RPW, int UNROLL>
static int launch_gemv32(const float* W, int64_t ldw, const float* X, int64_t ldx, float* Y, int64_t ldy,
                         int64_t ldy_inner, float* partial, int rows, int K, int m, int split_k, int sm_count,
                         cudaStream_t stream, int64_t* launches) {
  const int row_groups = (rows + RPW - 1) / RPW;
  const int warps = 8;
  int blocks = std::min((row_groups + warps - 1) / warps, sm_count * 8);
  int k_per_split = (K + split_k - 1) / split_k;
  k_per_split = (k_per_split + 127) / 128 * 128;
  gemv_f32_kernel<MRHS, RPW, UNROLL><<<dim3(blocks, split_k), warps * 32, 0, stream>>>(
      W, ldw, X, ldx, Y, ldy, ldy_inner, partial, rows, K, m, split_k, k_per_split);
  ++*launches;
  if (split_k > 1) {
    const int n = rows * m;
    gemv_f32_splitk_reduce_kernel<<<(n + 255) / 256, 256, 0, stream>>>(partial, Y, ldy, ldy_inner, rows, m, split_k);
    ++*launches;
  }
  return cudaGetLastError() == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

int gemv_f32_launch(const helix_cfg_t* cfg, const float* W, int64_t ldw, const float* X, int64_t ldx, float* Y,
                    int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes, int sm_count,
                    cudaStream_t stream, int64_t* launches) {
  if (!W || !X || !Y || rows <= 0 || K <= 0 || m <= 0 || m > 8) return HELIX_ERR_INVALID;
  if (ldw == 0) ldw = K;
  if (ldx == 0) ldx = K;
  if (ldy == 0) ldy = rows;
  if (ldy_inner == 0) ldy_inner = 1;
  if ((K & 3) || (ldw & 3) || (ldx & 3) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(X) & 15))
    return HELIX_ERR_ALIGN;
  const bool own = cfg && cfg->tile_m != 0;
  int split_k = (own && cfg->split_k > 0) ? cfg->split_k : gemv_f32_default_split(rows, K, sm_count);
  if (split_k > 1 && (K + split_k - 1) / split_k < 128) split_k = 1;
  const size_t need = gemv_f32_workspace_bytes(rows, m, split_k);
  if (need > 0 && (!ws || ws_bytes < need)) {
    if (own && cfg->split_k > 1) return HELIX_ERR_WORKSPACE;
    split_k = 1;
  }
  float* part = static_cast<float*>(ws);
  // tile_n = rows per warp (1 or 2), load_group = 16-byte loads in flight per row and thread (2, 4 or 8)
  const int rpw = (own && cfg->tile_n > 0) ? cfg->tile_n : (m <= 2 ? 2 : 1);
  const int unroll = (own && cfg->load_group > 0) ? cfg->load_group : (m <= 4 ? 4 : 2);
#define HELIX_GEMV32_CASE(MR, R, U)                                                                          \
  if (rpw == R && unroll == U)                                                                               \
    return launch_gemv32<MR, R, U>(W, ldw, X, ldx, Y, ldy, ldy_inner, part, rows, K, m, split_k, sm_count, stream, \
                                   launches);
#define HELIX_GEMV32_M(MR) \
  HELIX_GEMV32_CASE(MR, 1, 2) HELIX_GEMV32_CASE(MR, 1, 4) HELIX_GEMV32_CASE(MR, 1, 8) HELIX_GEMV32_CASE(MR, 2, 2) \
  HELIX_GEMV32_CASE(MR, 2, 4)
  if (m == 1) { HELIX_GEMV32_M(1) }
  else if (m == 2) { HELIX_GEMV32_M(2) }
  else if (m <= 4) { HELIX_GEMV32_M(4) }
  else { HELIX_GEMV32_M(8) }
#undef HELIX_GEMV32_M
#undef HELIX_GEMV32_CASE
  return HELIX_ERR_UNSUPPORTED;
}

}  // namespace helix
