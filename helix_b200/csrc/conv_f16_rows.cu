// 3 x 3, stride-1, pad-1 NHWC convolution, 64 -> 64 channels, with pixels on the accumulator rows and each item's input
// window resident in shared memory ("row pair" variant).
//
// The implicit-GEMM kernel in gemm_f16_tc.cu fetches every input pixel once per filter tap through the im2col tensor
// map; at 64 channels and 56 x 56 pixels that is 115 MB from L2 for a 12.8 MB input and bounds the layer at ~20 us
// (reference counterpart: src_template/Ampere_FP16/im2col.cu:37-97 materialises the same 9-fold copy in global
// memory).  Here a work item is two whole output rows of one image:
//   * its input window -- 4 padded rows of Wp = W + 2 pixels, 64 channels -- arrives with ONE tiled TMA box
//     (out-of-image pixels as zeros) as rows of 128 bytes, row q = h * Wp + w, 128-byte swizzled;
//   * accumulator row m is the padded position m = hl * Wp + wl of the row pair (2 Wp <= 128; positions wl >= W are
//     junk rows that are never stored), so the A operand of tap (r, s) is the SAME buffer read from row r * Wp + s
//     on: the tap only moves the start address of the matrix descriptor;
//   * all nine 64 x 64 weight slabs (72 KB) stay in shared memory for the life of the CTA;
//   * 36 MMAs of 128 x 64 x 16 per item; three issuing warps take the items round-robin, one accumulator each (a
//     128 x 64 MMA is bound by its operand fetch from shared memory, 48 cycles, and one warp cannot hand them over
//     that fast);
//   * the epilogue lays the two output rows out as 64 x 128-byte swizzled rows each and stores them with one TMA
//     store per output row (pixels beyond W are clipped by the tensor map).
// Each input row is read from L2 twice (once per neighbouring row pair) instead of nine times.
//
// Roles (256 threads, one CTA per SM, contiguous strips of items): warp 0 window loads, warps 1-3 MMA issue,
// warps 4-7 epilogue.  All waits are bounded.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "conv_common.cuh"
#include "kernels.h"

namespace helix {

namespace {

constexpr int kBM = 128;
constexpr int kCh = 64;               // input channels = output channels = one 128-byte row
constexpr int kThreads = 256;
constexpr int kTaps = 9;
constexpr int kWSlabBytes = kCh * kCh * 2;        // one tap's 64 x 64 weights
constexpr int kWinStages = 3;
constexpr int kWinBytes = 32768;                  // 4 rows x up to 64 padded pixels x 128 bytes
constexpr int kStageRowBytes = 64 * 128;          // one output row in the staging buffer: 64 pixel slots
constexpr int kStagingBytes = 2 * 2 * kStageRowBytes;   // two buffers of two output rows
constexpr int kAcc = 3;                           // accumulators = issuing warps = window stages: item i -> warp, accumulator
                                                  // and stage i % 3, so every barrier has ONE waiter that takes its phases in order
                                                  // (a waiter one phase ahead would mistake the barrier's initial state for its phase)
static_assert(kAcc == kWinStages, "one issuing warp per window stage");
constexpr int kTmemCols = 256;
constexpr int kEpiBar = 1;

struct RowsParams {
  int NB, H, W, Wp, Ho;
  int pairs;            // row pairs per image = ceil(Ho / 2)
  int items;            // NB * pairs
  int box_bytes;        // 4 * Wp * 128
  int independent;
  int probe;            // bit 0 = no MMAs, bit 1 = no window loads, bit 2 = no output stores
  int* status;
  FastDiv fd_pairs;
};

__global__ void __launch_bounds__(kThreads, 1)
conv_f16_rows_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                     const __grid_constant__ CUtensorMap tmap_y, const RowsParams p) {
  griddep_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;                                           // [9][64 x 128 bytes], swizzled
  uint8_t* sWin = sW + kTaps * kWSlabBytes;                     // [kWinStages][kWinBytes], swizzled rows
  uint8_t* sOut = sWin + kWinStages * kWinBytes;                // [2][2 rows][64 x 128 bytes]; also the reach of junk rows
  uint64_t* bars = reinterpret_cast<uint64_t*>(sOut + kStagingBytes);
  uint64_t* wbar = bars;                   // weights have landed
  uint64_t* full = bars + 1;               // [kWinStages] window of item i has landed
  uint64_t* done = bars + 1 + kWinStages;  // [kWinStages] MMAs of item i have completed
  uint64_t* tfull = bars + 1 + 2 * kWinStages;     // [kAcc]
  uint64_t* tempty = tfull + kAcc;                 // [kAcc]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tempty + kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // this CTA's strip of the (image, row pair) list
  const int t0 = (int)((int64_t)p.items * blockIdx.x / gridDim.x);
  const int t1 = (int)((int64_t)p.items * (blockIdx.x + 1) / gridDim.x);

  if (threadIdx.x == 0) {
    mbar_init(wbar, 1);
    for (int s = 0; s < kWinStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], 1);
    }
    for (int a = 0; a < kAcc; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_y);
  }
  if (warp == 1) tmem_alloc<kTmemCols>(tmem_ptr_smem);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  if (!p.independent) griddep_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ weights once, then one window per item
    if (lane == 0) {
      mbar_arrive_expect_tx(wbar, kTaps * kWSlabBytes);
      for (int t = 0; t < kTaps; ++t) tma_load_3d(sW + t * kWSlabBytes, &tmap_w, wbar, t * kCh, 0, 0);
      bool ok = true;
      int img, rp;
      fast_divmod(t0, p.fd_pairs, img, rp);
      for (int t = t0; ok && t < t1; ++t) {
        const int i = t - t0;
        const int s = i % kWinStages;
        ok = mbar_wait(&done[s], ((i / kWinStages) & 1) ^ 1, abort_flag, p.status);
        if (!ok) break;
        if (!(p.probe & 2)) {
          mbar_arrive_expect_tx(&full[s], (uint32_t)p.box_bytes);
          tma_load_4d(sWin + (size_t)s * kWinBytes, &tmap_x, &full[s], 0, -1, 2 * rp - 1, img);
        } else {
          mbar_arrive(&full[s]);
        }
        if (++rp == p.pairs) { rp = 0; ++img; }
      }
    }
  } else if (warp <= kAcc) {
    // ------------------------------------------------------------------ MMA issue (whole warp, one elected lane)
    // warp ME issues items ME, ME + 3, ... into accumulator ME
    const int ME = warp - 1;
    const uint32_t idesc = umma_idesc_f16(kBM, kCh);
    const uint32_t d_tmem = tmem_base + ME * kCh;
    const uint64_t w_desc0 = umma_desc_sw128(smem_u32(sW));
    const uint32_t win0 = smem_u32(sWin);
    const bool issue = !(p.probe & 1);
    bool ok = __all_sync(0xffffffffu, mbar_wait(wbar, 0, abort_flag, p.status));
    for (int i = ME; ok && t0 + i < t1; i += kAcc) {
      const int s = i % kWinStages;
      ok = __all_sync(0xffffffffu, mbar_wait(&tempty[ME], ((i / kAcc) & 1) ^ 1, abort_flag, p.status));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (i / kWinStages) & 1, abort_flag, p.status));
      if (!ok) break;
      tc_fence_after_sync();
      // The tensor core derives the swizzle phase of a row from the row's absolute shared-memory address, exactly as
      // the TMA did when it wrote the rows, so a window that starts at any row is described by its plain start address.
      const uint64_t a_desc0 = umma_desc_sw128(win0 + (uint32_t)s * kWinBytes);
      uint32_t tap_row16 = 0;      // first window row of the tap, in 16-byte units: (r * Wp + s) * 8
#pragma unroll
      for (int tap = 0; tap < kTaps; ++tap) {
        if (issue) {
#pragma unroll
          for (int k = 0; k < kCh / 16; ++k)
            umma_f16_ss_elect(d_tmem, a_desc0 + tap_row16 + 2 * k, w_desc0 + (uint32_t)(tap * (kWSlabBytes / 16)) + 2 * k,
                              idesc, (tap > 0) || (k > 0));
        }
        tap_row16 += 8u;
        if (tap % 3 == 2) tap_row16 += (uint32_t)(p.Wp - 3) * 8u;
      }
      umma_commit_elect(&done[s]);
      umma_commit_elect(&tfull[ME]);
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // TMEM lane = padded position q = hl * Wp + wl of the row pair, column = output channel.  The four warps lay the
    // two output rows out as 64 swizzled 128-byte rows each (pixel slot wl of row hl), then one thread stores each
    // output row with one TMA store; two staging buffers alternate.  The warps go on, or give up, together.
    const int quarter = warp & 3;
    const bool storer = warp == 4 && lane == 0;
    const int q = quarter * 32 + lane;
    const int hl = q >= p.Wp ? 1 : 0;
    const int wl = q - hl * p.Wp;
    const bool live = q < 2 * p.Wp;
    const uint32_t my_row = (uint32_t)(hl * 64 + wl) * 128u;
    bool ok = true;
    int img, rp;
    fast_divmod(t0, p.fd_pairs, img, rp);
    for (int t = t0; t < t1; ++t) {
      const int i = t - t0;
      const int acc = i % kAcc;
      ok = mbar_wait(&tfull[acc], (i / kAcc) & 1, abort_flag, p.status);
      ok = named_bar_and(kEpiBar, 128, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kCh;
      uint32_t lo[32], hi[32];
      tmem_ld_32x32b_x32(taddr, lo);
      tmem_ld_32x32b_x32(taddr + 32, hi);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (!(p.probe & 4)) {
        uint8_t* const buf = sOut + (size_t)(i & 1) * (2 * kStageRowBytes);
        if (storer) tma_store_wait_read_1();      // the stores of item i - 2 have left this buffer
        named_bar_sync(kEpiBar, 128);
        if (live) {
          const uint32_t row_base = smem_u32(buf) + my_row;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t* src = ch < 4 ? &lo[ch * 8] : &hi[(ch - 4) * 8];
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((ch ^ (wl & 7)) << 4)),
                         "r"(pack_half2(__uint_as_float(src[0]), __uint_as_float(src[1]))),
                         "r"(pack_half2(__uint_as_float(src[2]), __uint_as_float(src[3]))),
                         "r"(pack_half2(__uint_as_float(src[4]), __uint_as_float(src[5]))),
                         "r"(pack_half2(__uint_as_float(src[6]), __uint_as_float(src[7])))
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(kEpiBar, 128);
        if (storer) {
          const int ho = 2 * rp;
          tma_store_3d(&tmap_y, buf, 0, 0, img * p.Ho + ho);
          if (ho + 1 < p.Ho) tma_store_3d(&tmap_y, buf + kStageRowBytes, 0, 0, img * p.Ho + ho + 1);
          tma_store_commit();
        }
      }
      if (++rp == p.pairs) { rp = 0; ++img; }
    }
    if (storer) tma_store_wait_all();   // nothing of this thread's is in flight when the CTA tears down
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  // a launch that did not wait for its predecessor before its work waits for it now, so that completion order
  // along the stream stays transitive
  if (p.independent) griddep_wait();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

constexpr size_t kSmemBytes = 1024 + (size_t)kTaps * kWSlabBytes + (size_t)kWinStages * kWinBytes + kStagingBytes +
                              (1 + 2 * kWinStages + 2 * kAcc) * 8 + 16;

}  // namespace

// The geometry the kernel covers.  `worth_it`: also large and wide enough to beat the implicit-GEMM path (accumulator
// rows mostly live, at least a few items per SM).
bool conv_f16_rows_eligible(const ConvGeom& g, int sm_count, bool worth_it) {
  if (g.C != kCh || g.KO != kCh || g.R != 3 || g.S != 3 || g.stride != 1 || g.pad != 1) return false;
  if (g.W < 1 || g.W + 2 > 64 || g.H < 1 || g.Ho != g.H || g.Wo != g.W) return false;
  if ((int64_t)g.NB * ((g.Ho + 1) / 2) > 0x3fffffff) return false;
  if (worth_it && (g.W + 2 < 48 || (int64_t)g.NB * ((g.Ho + 1) / 2) < 3 * (int64_t)sm_count)) return false;
  return conv_tensor_map_encoder() != nullptr;
}

int conv_f16_rows_launch(const void* x, const void* w, void* y, const ConvGeom& g, int probe, int* status_dev,
                         int sm_count, bool independent, cudaStream_t stream, int64_t* launches) {
  if (!conv_f16_rows_eligible(g, sm_count, false)) return HELIX_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return HELIX_ERR_ALIGN;
  EncodeTiledFn fn = conv_tensor_map_encoder();
  if (!fn) return HELIX_ERR_CUDA;
  RowsParams p{};
  p.NB = g.NB; p.H = g.H; p.W = g.W; p.Wp = g.W + 2; p.Ho = g.Ho;
  p.pairs = (g.Ho + 1) / 2;
  p.items = g.NB * p.pairs;
  p.box_bytes = 4 * p.Wp * 128;
  p.independent = independent ? 1 : 0;
  p.probe = probe;
  p.status = status_dev;
  p.fd_pairs = make_fastdiv(p.pairs);
  CUtensorMap tx, tw, ty;
  {
    // activations x[N][H][W][64] as (C, W, H, N); one box = 64 channels x Wp pixels x 4 rows
    cuuint64_t dims[4] = {(cuuint64_t)kCh, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.NB};
    cuuint64_t strides[3] = {(cuuint64_t)kCh * 2, (cuuint64_t)g.W * kCh * 2, (cuuint64_t)g.H * g.W * kCh * 2};
    cuuint32_t box[4] = {(cuuint32_t)kCh, (cuuint32_t)p.Wp, 4, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  {
    // weights w[64][9 * 64] K-major; one box = 64 halves (one tap) x 64 output channels
    cuuint64_t dims[3] = {(cuuint64_t)kTaps * kCh, (cuuint64_t)kCh, 1};
    cuuint64_t strides[2] = {(cuuint64_t)kTaps * kCh * 2, (cuuint64_t)kTaps * kCh * kCh * 2};
    cuuint32_t box[3] = {(cuuint32_t)kCh, (cuuint32_t)kCh, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  {
    // y[N][Ho][Wo][64] as (64, Wo, N * Ho); one box = one output row, 64 pixel slots of which Wo exist
    cuuint64_t dims[3] = {(cuuint64_t)kCh, (cuuint64_t)g.Wo, (cuuint64_t)g.NB * g.Ho};
    cuuint64_t strides[2] = {(cuuint64_t)kCh * 2, (cuuint64_t)g.Wo * kCh * 2};
    cuuint32_t box[3] = {(cuuint32_t)kCh, 64, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&ty, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  auto kern = conv_f16_rows_kernel;
  {
    static std::mutex mu;
    static bool granted[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !granted[dev]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
        return HELIX_ERR_CUDA;
      granted[dev] = true;
    }
  }
  const int grid = (int)std::min<int64_t>(p.items, sm_count);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = kSmemBytes;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, tx, tw, ty, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, kSmemBytes, stream>>>(tx, tw, ty, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  return HELIX_OK;
}

}  // namespace helix
