// Memory-bound fp16 GEMV for 1..8 right-hand sides (non tensor core).
//
//   Y[i, r] = sum_k W[r, k] * X[i, k]        W: rows x K (row-major, the HBM stream)
//                                              X: m x K, m <= 8 (stays in L1/L2)
// fp32 accumulate, one rounding to half at the end.  Counterpart of the reference's
// mySGemvKernel_Stage4 (src_template/Ampere_FP16/gemv.cu:151-216) and its split-K twin
// (gemv_splitK.cu:153-221); unlike those it accumulates in fp32, takes any row count and any
// K that is a multiple of 8, and reduces split-K partials deterministically.
//
// Mapping: one warp owns RPW consecutive rows; lane l reads the 16-byte chunk l of each
// 512-byte row segment, UNROLL segments in flight per row, so a thread keeps RPW*UNROLL
// independent 128-bit streaming loads outstanding.  Lanes are reduced with a shuffle tree.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace helix {

template <int MRHS, int RPW, int UNROLL>
__global__ void __launch_bounds__(256)
gemv_f16_kernel(const __half* __restrict__ W, int64_t ldw, const __half* __restrict__ X, int64_t ldx,
                __half* __restrict__ Y, int64_t ldy, int64_t ldy_inner, float* __restrict__ partial,
                int rows, int K, int m, int split_k, int k_per_split, int order_mode) {
  // Let the next kernel on the stream be scheduled while this one drains.  How this launch orders
  // itself after the kernel queued before it (order_mode):
  //   0  wait for it before touching global memory (safe default);
  //   1  W is not written by it (weights): the first batch of W loads is issued, THEN the kernel
  //      waits, then reads X and later writes Y -- launch latency and ramp-up hide behind the
  //      predecessor's tail while X may still be its output;
  //   2  nothing is shared with it: no wait before the work.
  // In modes 1 and 2 every thread that has not waited yet does so just before it exits, after its last
  // store: this kernel then cannot complete before its predecessor has, so a later kernel that waits
  // for this one is still ordered after everything queued earlier.
  griddep_launch_dependents();
  bool waited = order_mode == 0;
  if (order_mode == 0) griddep_wait();
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

    const __half* wrow[RPW];
#pragma unroll
    for (int r = 0; r < RPW; ++r) wrow[r] = W + (int64_t)min(r0 + r, rows - 1) * ldw;

    for (int k0 = k_begin + lane * 8; k0 < k_end; k0 += 256 * UNROLL) {
      uint4 wv[UNROLL][RPW];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = k0 + u * 256;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          if (k < k_end) wv[u][r] = ldg_stream_16(wrow[r] + k);
          else wv[u][r] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (!waited && order_mode == 1) {   // warp-uniform
        griddep_wait();
        waited = true;
      }
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int k = k0 + u * 256;
        if (k < k_end) {
#pragma unroll
          for (int i = 0; i < MRHS; ++i) {
            if (i < m) {
              const uint4 xv = __ldg(reinterpret_cast<const uint4*>(X + (int64_t)i * ldx + k));
              const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
              for (int r = 0; r < RPW; ++r) {
                const __half2* wh = reinterpret_cast<const __half2*>(&wv[u][r]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 wf = __half22float2(wh[j]);
                  const float2 xf = __half22float2(xh[j]);
                  acc[r][i] = fmaf(wf.x, xf.x, acc[r][i]);
                  acc[r][i] = fmaf(wf.y, xf.y, acc[r][i]);
                }
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
    if (!waited && order_mode == 1) {   // empty K range: still order the stores after the predecessor
      griddep_wait();
      waited = true;
    }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        if (r0 + r < rows) {
#pragma unroll
          for (int i = 0; i < MRHS; ++i) {
            if (i < m) {
              if (split_k == 1) Y[(int64_t)i * ldy + (int64_t)(r0 + r) * ldy_inner] = __float2half_rn(acc[r][i]);
              else partial[((int64_t)ks * m + i) * rows + r0 + r] = acc[r][i];
            }
          }
        }
      }
    }
  }
  if (!waited) griddep_wait();
}

// Sums the split-K partials in slice order (deterministic) and rounds once.
__global__ void gemv_splitk_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ Y, int64_t ldy,
                                          int64_t ldy_inner, int rows, int m, int split_k) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * m) return;
  const int i = idx / rows, r = idx - i * rows;
  float s = 0.0f;
  for (int ks = 0; ks < split_k; ++ks) s += partial[((int64_t)ks * m + i) * rows + r];
  Y[(int64_t)i * ldy + (int64_t)r * ldy_inner] = __float2half_rn(s);
}

size_t gemv_f16_workspace_bytes(int rows, int m, int split_k) {
  return split_k > 1 ? (size_t)split_k * m * rows * sizeof(float) : 0;
}

int gemv_f16_default_split(int rows, int K, int sm_count) {
  // Cut K only when there are too few rows to keep enough bytes in flight: a warp holds 4 KiB of loads, and
  // the stream needs some 24 warps per SM before HBM saturates (512 rows x 500 000: split 4 reads at 2.9 TB/s,
  // split 16 at 6.5).  The partials cost a second launch and forbid overlapping with the neighbouring
  // launches, so beyond four warps per SM only very long rows are cut.
  const int groups = (rows + 1) / 2;
  int split = 1;
  while (split < 16 && K / (split * 2) >= 2048 &&
         ((int64_t)groups * split < (int64_t)sm_count * 4 ||
          ((int64_t)groups * split < (int64_t)sm_count * 24 && K / (split * 2) >= 16384)))
    split *= 2;
  return split;
}

// Set by gemv_f16_launch for the duration of one call: how the launch orders itself after the
// kernel queued before it (see order_mode in the kernel).
static thread_local int independent = 0;

template <int MRHS, int RPW, int UNROLL>
static int launch_gemv(const __half* W, int64_t ldw, const __half* X, int64_t ldx, __half* Y, int64_t ldy,
                       int64_t ldy_inner, float* partial, int rows, int K, int m, int split_k, int sm_count,
                       cudaStream_t stream, int64_t* launches) {
  const int row_groups = (rows + RPW - 1) / RPW;
  const int warps = 8;
  int blocks = (row_groups + warps - 1) / warps;
  const int max_blocks = sm_count * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  int k_per_split = (K + split_k - 1) / split_k;
  k_per_split = (k_per_split + 255) / 256 * 256;
  dim3 grid(blocks, split_k);
  // split-K shares its scratch with neighbouring launches, so it always orders itself after them
  const int indep = split_k == 1 ? independent : 0;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = grid;
  lc.blockDim = dim3(warps * 32);
  lc.dynamicSmemBytes = 0;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  if (cudaLaunchKernelEx(&lc, gemv_f16_kernel<MRHS, RPW, UNROLL>, W, ldw, X, ldx, Y, ldy, ldy_inner, partial, rows, K,
                         m, split_k, k_per_split, indep) != cudaSuccess) {
    (void)cudaGetLastError();
    gemv_f16_kernel<MRHS, RPW, UNROLL><<<grid, warps * 32, 0, stream>>>(W, ldw, X, ldx, Y, ldy, ldy_inner, partial,
                                                                        rows, K, m, split_k, k_per_split, indep);
  }
  ++*launches;
  if (split_k > 1) {
    const int n = rows * m;
    gemv_splitk_reduce_kernel<<<(n + 255) / 256, 256, 0, stream>>>(partial, Y, ldy, ldy_inner, rows, m, split_k);
    ++*launches;
  }
  return cudaGetLastError() == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

// (rows per warp, 16-byte loads in flight per row and thread) variants compiled in.
template <int MRHS>
static int launch_gemv_variant(int rpw, int unroll, const __half* W, int64_t ldw, const __half* X, int64_t ldx,
                               __half* Y, int64_t ldy, int64_t ldy_inner, float* partial, int rows, int K, int m,
                               int split_k, int sm_count, cudaStream_t stream, int64_t* launches) {
#define HELIX_GEMV_CASE(R, U)                                                                                 \
  if (rpw == R && unroll == U)                                                                                \
    return launch_gemv<MRHS, R, U>(W, ldw, X, ldx, Y, ldy, ldy_inner, partial, rows, K, m, split_k, sm_count, \
                                   stream, launches);
  HELIX_GEMV_CASE(1, 2)
  HELIX_GEMV_CASE(1, 4)
  HELIX_GEMV_CASE(1, 8)
  HELIX_GEMV_CASE(1, 16)
  HELIX_GEMV_CASE(2, 2)
  HELIX_GEMV_CASE(2, 4)
  HELIX_GEMV_CASE(2, 8)
#undef HELIX_GEMV_CASE
  return HELIX_ERR_UNSUPPORTED;
}

int gemv_f16_launch(const helix_cfg_t* cfg, const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y,
                    int64_t ldy, int64_t ldy_inner, int rows, int K, int m, void* ws, size_t ws_bytes,
                    int sm_count, int order_mode, cudaStream_t stream, int64_t* launches) {
  struct Scope {
    explicit Scope(int v) { independent = v; }
    ~Scope() { independent = 0; }
  } scope(order_mode);
  if (!W || !X || !Y || rows <= 0 || K <= 0 || m <= 0 || m > 8) return HELIX_ERR_INVALID;
  if (ldw == 0) ldw = K;
  if (ldx == 0) ldx = K;
  if (ldy == 0) ldy = rows;
  if (ldy_inner == 0) ldy_inner = 1;
  if ((K & 7) || (ldw & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(X) & 15))
    return HELIX_ERR_ALIGN;
  int split_k = (cfg && cfg->tile_m != 0 && cfg->split_k > 0) ? cfg->split_k
                                                              : gemv_f16_default_split(rows, K, sm_count);
  if (split_k > 1 && (K + split_k - 1) / split_k < 256) split_k = 1;
  const size_t need = gemv_f16_workspace_bytes(rows, m, split_k);
  if (need > 0 && (!ws || ws_bytes < need)) {
    if (cfg && cfg->tile_m != 0 && cfg->split_k > 1) return HELIX_ERR_WORKSPACE;
    split_k = 1;  // automatic choice falls back to the workspace-free variant
  }
  const __half* w = static_cast<const __half*>(W);
  const __half* x = static_cast<const __half*>(X);
  __half* y = static_cast<__half*>(Y);
  float* part = static_cast<float*>(ws);
  // tile_n = rows per warp, load_group = loads in flight per row; defaults favour deep
  // memory-level parallelism (one pass over K per warp where K allows)
  int rpw = (cfg && cfg->tile_m != 0 && cfg->tile_n > 0) ? cfg->tile_n : (m <= 2 ? 2 : 1);
  int unroll = (cfg && cfg->tile_m != 0 && cfg->load_group > 0) ? cfg->load_group : (m <= 4 ? 4 : 2);
  if (m == 1) return launch_gemv_variant<1>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, part, rows, K, m, split_k, sm_count, stream, launches);
  if (m == 2) return launch_gemv_variant<2>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, part, rows, K, m, split_k, sm_count, stream, launches);
  if (m <= 4) return launch_gemv_variant<4>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, part, rows, K, m, split_k, sm_count, stream, launches);
  return launch_gemv_variant<8>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, part, rows, K, m, split_k, sm_count, stream, launches);
}

// ---------------------------------------------------------------------------------------------
// Split-K GEMV whose partial sums live in a buffer that is part of the library image.
//
// Some users of this library may not create device memory at the moment they need a GEMV: a
// decode loop that has handed every byte of HBM to its own pool cannot call cudaMalloc (it may
// fail, and it synchronises the device).  For them the fp32 partials of the split-K variant are
// kept in the fixed array below instead of a caller-supplied workspace.  Every GPU on which the
// library is loaded carries these 4 MiB until the process exits.
//
// In host code the name `g_gemv_static_scratch` is only a handle for the symbol, not an address
// the GPU understands; the device address is looked up once per device with
// cudaGetSymbolAddress (that device being current) and that pointer is what the kernels get.
constexpr size_t kGemvStaticFloats = size_t(1) << 20;  // 4 MiB of fp32 partials
static __device__ __align__(256) float g_gemv_static_scratch[kGemvStaticFloats];

size_t gemv_f16_static_capacity_floats() { return kGemvStaticFloats; }

// The set-up (symbol lookup) happens in the first call made on each device, so that first call
// should come before any stream capture.  All calls share the one array: it still holds
// the previous call's partials when a call starts, which is harmless because the kernel writes
// every slot the reduction reads before it is read (nothing has to start at zero) -- but two
// calls that may run on the GPU at the same time (different streams) would overwrite each
// other's partials, so callers must order them.  Nothing here allocates or frees memory.
int gemv_f16_static_launch(const void* W, int64_t ldw, const void* X, int64_t ldx, void* Y, int64_t ldy,
                           int64_t ldy_inner, int rows, int K, int m, int split_k, int sm_count,
                           cudaStream_t stream, int64_t* launches) {
  if (!W || !X || !Y || rows <= 0 || K <= 0 || m <= 0 || m > 8 || split_k < 1) return HELIX_ERR_INVALID;
  if (ldw == 0) ldw = K;
  if (ldx == 0) ldx = K;
  if (ldy == 0) ldy = rows;
  if (ldy_inner == 0) ldy_inner = 1;
  if ((K & 7) || (ldw & 7) || (ldx & 7) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(X) & 15))
    return HELIX_ERR_ALIGN;
  if (split_k > 1 && (K + split_k - 1) / split_k < 256) split_k = 1;
  // a single pass over K (split_k = 1, asked for or after the clamp above) never touches the array
  if (split_k > 1 && (size_t)split_k * (size_t)m * (size_t)rows > kGemvStaticFloats) return HELIX_ERR_CAPACITY;

  static std::mutex mu;
  static float* scratch_on_device[64] = {nullptr};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HELIX_ERR_NODEVICE;
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_on_device[dev]) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_gemv_static_scratch) != cudaSuccess || !p) return HELIX_ERR_CUDA;
      scratch_on_device[dev] = static_cast<float*>(p);
    }
    scratch = scratch_on_device[dev];
  }
  const __half* w = static_cast<const __half*>(W);
  const __half* x = static_cast<const __half*>(X);
  __half* y = static_cast<__half*>(Y);
  const int rpw = m <= 2 ? 2 : 1;
  const int unroll = m <= 4 ? 4 : 2;
  if (m == 1) return launch_gemv_variant<1>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, scratch, rows, K, m, split_k, sm_count, stream, launches);
  if (m == 2) return launch_gemv_variant<2>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, scratch, rows, K, m, split_k, sm_count, stream, launches);
  if (m <= 4) return launch_gemv_variant<4>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, scratch, rows, K, m, split_k, sm_count, stream, launches);
  return launch_gemv_variant<8>(rpw, unroll, w, ldw, x, ldx, y, ldy, ldy_inner, scratch, rows, K, m, split_k, sm_count, stream, launches);
}

}  // namespace helix
