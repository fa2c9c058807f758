// True-fp32 NHWC convolution = column matrix + FFMA GEMM.
//
// The reference's fp32 convolution is an explicit im2col (src_template/Ampere_FP32/im2col.cu:37-97,
// NCHW) followed by its SIMT GEMM on M = B*Ho*Wo, N = OC, K = IC*kH*kW
// (scripts/Ampere_FP32/Ampere_FP32_conv.py:101-113).  Same decomposition here for NHWC: one kernel
// writes the column matrix col[M][R*S*C] (k ordered (r, s, c), zeros where the window leaves the
// image), one transposes the weights w[KO][R][S][C] to wt[R*S*C][KO], and sgemm_f32 computes
// y[M][KO] = col x wt with its usual guarantee (every output one fmaf chain over ascending k).  A
// 1x1, stride-1, unpadded convolution uses x itself as the column matrix.  Both matrices live in the
// caller's workspace.
#include "common.cuh"
#include "kernels.h"

namespace helix {

struct Im2colDivs { FastDiv cq, s, r, wo, ho; };

// One thread per 4 consecutive channels (VEC) or per element of the column matrix.  With fewer than
// 2^31 work items (SMALL) the index is split with multiply-high reciprocals instead of 64-bit divisions.
template <bool VEC, bool SMALL>
__global__ void __launch_bounds__(256) im2col_f32_nhwc_kernel(const float* __restrict__ x, float* __restrict__ col,
                                                              int H, int W, int C, int R, int S, int stride, int pad,
                                                              int Ho, int Wo, int64_t total, Im2colDivs dv) {
  constexpr int E = VEC ? 4 : 1;
  const int cq = C / E;                       // channel groups per tap
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int c, s, r, wo, ho;
    int64_t t, n;                              // t = output pixel index m
    if (SMALL) {
      int q, rem, t32, t2, n32;
      fast_divmod((int)i, dv.cq, q, rem); c = rem * E;
      fast_divmod(q, dv.s, q, s);
      fast_divmod(q, dv.r, t32, r);
      fast_divmod(t32, dv.wo, t2, wo);
      fast_divmod(t2, dv.ho, n32, ho);
      t = t32; n = n32;
    } else {
      c = (int)(i % cq) * E;
      t = i / cq;
      s = (int)(t % S); t /= S;
      r = (int)(t % R); t /= R;
      wo = (int)(t % Wo);
      const int64_t t2 = t / Wo;
      ho = (int)(t2 % Ho);
      n = t2 / Ho;
    }
    const int h = ho * stride - pad + r, w = wo * stride - pad + s;
    const bool inside = h >= 0 && h < H && w >= 0 && w < W;
    float* dst = col + (t * R * S + (int64_t)r * S + s) * C + c;
    if (VEC) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (inside) v = *reinterpret_cast<const float4*>(x + ((n * H + h) * W + w) * C + c);
      *reinterpret_cast<float4*>(dst) = v;
    } else {
      *dst = inside ? x[((n * H + h) * W + w) * C + c] : 0.0f;
    }
  }
}

// wt[k][o] = w[o][k] through a 32 x 33 shared tile.
__global__ void __launch_bounds__(256) transpose_f32_kernel(const float* __restrict__ w, float* __restrict__ wt,
                                                            int rows, int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int j = ty; j < 32; j += 8)
    if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = w[(int64_t)(r0 + j) * cols + c0 + tx];
  __syncthreads();
  for (int j = ty; j < 32; j += 8)
    if (c0 + j < cols && r0 + tx < rows) wt[(int64_t)(c0 + j) * rows + r0 + tx] = tile[tx][j];
}

static inline size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

static bool conv_f32_is_gemm(const ConvGeom& g) { return g.R == 1 && g.S == 1 && g.stride == 1 && g.pad == 0; }

size_t conv_f32_workspace_bytes(const ConvGeom& g) {
  const int64_t M = (int64_t)g.NB * g.Ho * g.Wo, K = (int64_t)g.R * g.S * g.C;
  if (M <= 0 || K <= 0 || g.KO <= 0) return 0;
  const size_t col = conv_f32_is_gemm(g) ? 0 : align256((size_t)M * K * sizeof(float));
  return col + align256((size_t)K * g.KO * sizeof(float));
}

int conv_f32_launch(const helix_cfg_t* cfg, const float* x, const float* w, float* y, const ConvGeom& g, void* ws,
                    size_t ws_bytes, int sm_count, cudaStream_t stream, int64_t* launches) {
  if (!x || !w || !y || g.NB <= 0 || g.H <= 0 || g.W <= 0 || g.C <= 0 || g.KO <= 0 || g.R <= 0 || g.S <= 0 ||
      g.stride <= 0 || g.pad < 0 || g.Ho <= 0 || g.Wo <= 0)
    return HELIX_ERR_INVALID;
  const int64_t M64 = (int64_t)g.NB * g.Ho * g.Wo, K64 = (int64_t)g.R * g.S * g.C;
  if (M64 > 0x7fffffff || K64 > 0x7fffffff) return HELIX_ERR_INVALID;
  const int M = (int)M64, K = (int)K64;
  const size_t need = conv_f32_workspace_bytes(g);
  if (!ws || ws_bytes < need) return HELIX_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(ws) & 255) return HELIX_ERR_ALIGN;
  const bool as_gemm = conv_f32_is_gemm(g);
  float* col = static_cast<float*>(ws);
  float* wt = reinterpret_cast<float*>(static_cast<char*>(ws) + (as_gemm ? 0 : align256((size_t)M * K * sizeof(float))));
  {
    dim3 grid((K + 31) / 32, (g.KO + 31) / 32);
    transpose_f32_kernel<<<grid, 256, 0, stream>>>(w, wt, g.KO, K);
    ++*launches;
  }
  const float* a = x;
  if (!as_gemm) {
    const bool vec = (g.C % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int64_t total = (int64_t)M * g.R * g.S * (vec ? g.C / 4 : g.C);
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)sm_count * 16);
    const bool small = total < (int64_t)0x7fffffff;
    Im2colDivs dv{make_fastdiv(vec ? g.C / 4 : g.C), make_fastdiv(g.S), make_fastdiv(g.R), make_fastdiv(g.Wo),
                  make_fastdiv(g.Ho)};
#define HELIX_IM2COL(V, SM)                                                                                        \
  im2col_f32_nhwc_kernel<V, SM><<<blocks, 256, 0, stream>>>(x, col, g.H, g.W, g.C, g.R, g.S, g.stride, g.pad, g.Ho, \
                                                            g.Wo, total, dv)
    if (vec && small) HELIX_IM2COL(true, true);
    else if (vec) HELIX_IM2COL(true, false);
    else if (small) HELIX_IM2COL(false, true);
    else HELIX_IM2COL(false, false);
#undef HELIX_IM2COL
    ++*launches;
    a = col;
  }
  if (cudaGetLastError() != cudaSuccess) return HELIX_ERR_CUDA;
  return sgemm_f32_launch(cfg, a, K, 0, wt, g.KO, y, g.KO, M, g.KO, K, sm_count, stream, launches);
}

}  // namespace helix
