// Stride-1 NHWC convolution with the input window resident in shared memory ("halo" variant).
//
// The implicit-GEMM kernel in gemm_f16_tc.cu fetches every input pixel once per filter tap
// (R*S times) and every weight slab once per 128 output pixels, and is bound by that operand
// traffic (reference counterpart: src_template/Ampere_FP16/im2col.cu:37-97 materialises the
// R*S-fold copy in global memory).  Here a work item is a block of TH whole output rows of one
// image.  Its input window -- TH + R - 1 padded rows of Wp = W + 2*pad pixels, 64 channels -- is
// brought in by ONE tiled TMA box per channel block (out-of-image pixels arrive as zeros) and laid
// out as rows of 128 bytes, row index q = h*Wp + w, 128-byte swizzled.  The GEMM M axis runs over
// the padded positions q = hl*Wp + wl of the block (wl >= Wo are junk rows that are never stored),
// so the A operand of filter tap (r, s) is the SAME buffer read from row r*Wp + s on: the tap only
// moves the start address of the shared-memory matrix descriptor.  Each input byte is loaded once
// per item instead of R*S times, and one weight slab feeds two row blocks (two accumulators), which
// halves the weight traffic per output as well.
//
// Roles (256 threads): warp 0 window loads, warps 1-2 weight-slab loads (alternating slabs),
// warp 3 MMA issue + TMEM allocation, warps 4-7 epilogue.  All waits are bounded.
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace helix {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kThreads = 288;     // warp 8: second MMA issuer
constexpr int kHaloStages = 2;     // windows in flight (each holds up to two row blocks)
constexpr int kMaxBStages = 8;
constexpr int kBWarps = 2;

struct HaloParams {
  __half* y;
  int KO, NB, H, W, C, Ho, Wo, R, S, pad;
  int Wp;            // padded row length = W + 2 * pad
  int TH;            // output rows per block, TH * Wp <= 128
  int HR;            // input rows per block = TH + R - 1
  int RB;            // row blocks per image
  int blocks;        // NB * RB
  int pairs;         // ceil(blocks / 2)
  int tiles_n;
  int items;         // pairs * tiles_n
  int cblocks;       // C / 64
  int taps;          // R * S
  int buf_bytes;     // bytes of one block's window buffer (multiple of 1024)
  int box_bytes;     // bytes one window box delivers = HR * Wp * 128
  int b_stages;
  int independent;
  int vec_ok;        // 16-byte output stores are possible
  int probe;         // tuning instrument (helix_cfg_t.probe): 1 = issue no MMA
  int* status;
  FastDiv fd_tiles_n, fd_rb, fd_wp, fd_s;
  unsigned long long* trace;   // optional per-CTA timeline (null = off), same layout as the GEMM kernels
};

__device__ __forceinline__ void htrace(const HaloParams& p, int word) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * kTraceWords + word] = (unsigned long long)clock64();
}
__device__ __forceinline__ void htrace_item(const HaloParams& p, int idx, int slot) {
  if (idx < kTraceTiles) htrace(p, 8 + idx * 6 + slot);
}
__device__ __forceinline__ void htrace_slab(const HaloParams& p, int which, int n) {
  if (n < kTraceSlabs) htrace(p, 8 + 6 * kTraceTiles + which * kTraceSlabs + n);
}

struct HaloItem {
  int nb;            // output-channel tile
  int nsub;          // 1 or 2 row blocks
  int img[2], ho0[2];
};

__device__ __forceinline__ bool halo_item(const HaloParams& p, int t, HaloItem& it) {
  if (t >= p.items) return false;
  int pr;
  fast_divmod(t, p.fd_tiles_n, pr, it.nb);
  it.nsub = (2 * pr + 1 < p.blocks) ? 2 : 1;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const int u = min(2 * pr + s, p.blocks - 1);
    int rb;
    fast_divmod(u, p.fd_rb, it.img[s], rb);
    it.ho0[s] = rb * p.TH;
  }
  return true;
}

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

// Descriptor of a 128-byte-swizzled K-major operand whose first row is not at the start of a
// 1024-byte swizzle atom.  The tensor core derives the XOR phase of a row from the row's absolute
// shared-memory address (bits [7,10)), exactly as the TMA did when it wrote the rows, so the plain
// descriptor is right; the base-offset field (bits [49,52)) must stay zero -- measured: filling it
// with the start row's phase makes the hardware subtract that phase again.
__device__ __forceinline__ uint64_t umma_desc_sw128_rows(uint32_t smem_addr) {
  return umma_desc_sw128(smem_addr);
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_f16_halo_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                     const HaloParams p) {
  constexpr int kBBytes = BN * kBK * 2;
  constexpr int kTmemCols = 4 * BN <= 256 ? 256 : 512;   // two accumulators per item, double buffered
  constexpr uint32_t kIdesc = umma_idesc_f16(kBM, BN);

  griddep_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sH = smem;                                                  // [kHaloStages][2][buf_bytes]
  uint8_t* sB = smem + (size_t)kHaloStages * 2 * p.buf_bytes;         // [b_stages][kBBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + (size_t)p.b_stages * kBBytes);
  uint64_t* hfull = bars;            // [2]
  uint64_t* hempty = bars + 2;       // [2]
  uint64_t* bfull = bars + 4;        // [8]
  uint64_t* bempty = bars + 12;      // [8]
  uint64_t* tfull = bars + 20;       // [2]
  uint64_t* tempty = bars + 22;      // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int grid = gridDim.x;

  if (threadIdx.x == 0) {
    if (p.trace != nullptr) {
      p.trace[(size_t)blockIdx.x * kTraceWords + 0] = global_timer_ns();
      htrace(p, 1);
    }
    for (int s = 0; s < kHaloStages; ++s) {
      mbar_init(&hfull[s], 1);
      mbar_init(&hempty[s], 2);
    }
    for (int s = 0; s < p.b_stages; ++s) {
      mbar_init(&bfull[s], 1);
      mbar_init(&bempty[s], 2);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 2);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  if (warp == 3) tmem_alloc<kTmemCols>(tmem_ptr_smem);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (!p.independent) griddep_wait();
  if (threadIdx.x == 0) htrace(p, 2);

  if (warp == 0) {
    // ------------------------------------------------------------------ window loads
    if (lane == 0) {
      bool ok = true;
      int n = 0;   // window sequence number: one per (item, channel block)
      HaloItem it;
      int idx = 0;
      for (int t = cta; ok && halo_item(p, t, it); t += grid, ++idx) {
        for (int cb = 0; cb < p.cblocks && ok; ++cb, ++n) {
          const int hs = n % kHaloStages;
          const uint32_t ph = (uint32_t)(n / kHaloStages) & 1u;
          ok = mbar_wait(&hempty[hs], ph ^ 1, abort_flag, p.status);
          if (!ok) break;
          htrace_item(p, idx, cb == 0 ? 0 : 1);
          mbar_arrive_expect_tx(&hfull[hs], (uint32_t)(it.nsub * p.box_bytes));
          for (int s = 0; s < it.nsub; ++s)
            tma_load_4d(sH + ((size_t)hs * 2 + s) * p.buf_bytes, &tmap_x, &hfull[hs], cb * kBK, -p.pad,
                        it.ho0[s] - p.pad, it.img[s]);
        }
      }
    }
  } else if (warp <= kBWarps) {
    // ------------------------------------------------------------------ weight-slab loads
    // slab sequence: for each item, for each channel block, for each tap; slab n belongs to
    // issuer n % kBWarps (an issuing thread is held a few hundred cycles per tensor copy)
    const int issuer = warp - 1;
    if (lane == 0 && issuer < min(kBWarps, p.b_stages)) {
      const int nissue = min(kBWarps, p.b_stages);
      bool ok = true;
      int n = 0;
      HaloItem it;
      for (int t = cta; ok && halo_item(p, t, it); t += grid) {
        for (int cb = 0; cb < p.cblocks && ok; ++cb) {
          for (int tap = 0; tap < p.taps; ++tap, ++n) {
            if (n % nissue != issuer) continue;
            const int bs = n % p.b_stages;
            const uint32_t ph = (uint32_t)(n / p.b_stages) & 1u;
            ok = mbar_wait(&bempty[bs], ph ^ 1, abort_flag, p.status);
            if (!ok) break;
            htrace_slab(p, 0, n);
            mbar_arrive_expect_tx(&bfull[bs], kBBytes);
            tma_load_3d(sB + (size_t)bs * kBBytes, &tmap_w, &bfull[bs], tap * p.C + cb * kBK, it.nb * BN, 0);
          }
        }
      }
    }
  } else if (warp == 3 || warp == 8) {
    // ------------------------------------------------------------------ MMA issuers: one per row block
    const int my_sub = warp == 3 ? 0 : 1;
    if (lane == 0) {
      bool ok = true;
      int hn = 0, bn_seq = 0, idx = 0;
      HaloItem it;
      for (int t = cta; ok && halo_item(p, t, it); t += grid, ++idx) {
        const int acc = idx & 1;
        const uint32_t acc_phase = (idx >> 1) & 1;
        ok = mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        htrace_item(p, idx, 2);
        const uint32_t d_tmem = tmem_base + acc * (2 * BN);
        for (int cb = 0; cb < p.cblocks && ok; ++cb, ++hn) {
          const int hs = hn % kHaloStages;
          ok = mbar_wait(&hfull[hs], (uint32_t)(hn / kHaloStages) & 1u, abort_flag, p.status);
          if (!ok) break;
          const uint32_t win0 = smem_u32(sH + (size_t)hs * 2 * p.buf_bytes);
          int fr = 0, fs = 0;
          for (int tap = 0; tap < p.taps; ++tap, ++bn_seq) {
            const int bs = bn_seq % p.b_stages;
            ok = mbar_wait(&bfull[bs], (uint32_t)(bn_seq / p.b_stages) & 1u, abort_flag, p.status);
            if (!ok) break;
            htrace_slab(p, 1, bn_seq);
            tc_fence_after_sync();
            const uint64_t db = umma_desc_sw128(smem_u32(sB + (size_t)bs * kBBytes));
            const uint32_t shift = (uint32_t)(fr * p.Wp + fs) * 128u;   // first row of this tap's window
            // the two row blocks' accumulators alternate: consecutive MMAs into the same accumulator
            // wait for one another, independent ones overlap
            if (my_sub < it.nsub && !(p.probe & 1)) {
              const uint64_t da = umma_desc_sw128_rows(win0 + (uint32_t)my_sub * p.buf_bytes + shift);
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k)
                umma_f16_ss(d_tmem + my_sub * BN, da + 2 * k, db + 2 * k, kIdesc, (cb > 0) || (tap > 0) || (k > 0));
            }
            umma_commit(&bempty[bs]);
            if (++fs == p.S) { fs = 0; ++fr; }
          }
          if (ok) umma_commit(&hempty[hs]);
        }
        if (ok) umma_commit(&tfull[acc]);
        htrace_item(p, idx, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    bool ok = true;
    int idx = 0;
    HaloItem it;
    const int q = quarter * 32 + lane;          // padded position inside the block
    int hl, wl;
    fast_divmod(q, p.fd_wp, hl, wl);
    for (int t = cta; ok && halo_item(p, t, it); t += grid, ++idx) {
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      ok = mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      if (quarter == 0 && lane == 0) htrace_item(p, idx, 4);
      for (int s = 0; s < it.nsub; ++s) {
        const int ho = it.ho0[s] + hl;
        const bool valid = hl < p.TH && ho < p.Ho && wl < p.Wo;
        __half* dst = p.y + (((int64_t)it.img[s] * p.Ho + ho) * p.Wo + wl) * p.KO + it.nb * BN;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (2 * BN) + s * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c0, r);
          tmem_ld_wait();
          const int col0 = it.nb * BN + c0;
          if (valid && col0 < p.KO) {
#pragma unroll
            for (int jj = 0; jj < 32; jj += 8) {
              if (p.vec_ok && col0 + jj + 8 <= p.KO) {
                __half2 h0 = __floats2half2_rn(__uint_as_float(r[jj + 0]), __uint_as_float(r[jj + 1]));
                __half2 h1 = __floats2half2_rn(__uint_as_float(r[jj + 2]), __uint_as_float(r[jj + 3]));
                __half2 h2 = __floats2half2_rn(__uint_as_float(r[jj + 4]), __uint_as_float(r[jj + 5]));
                __half2 h3 = __floats2half2_rn(__uint_as_float(r[jj + 6]), __uint_as_float(r[jj + 7]));
                uint4 v;
                v.x = *reinterpret_cast<uint32_t*>(&h0);
                v.y = *reinterpret_cast<uint32_t*>(&h1);
                v.z = *reinterpret_cast<uint32_t*>(&h2);
                v.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + c0 + jj) = v;
              } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                  if (col0 + jj + e < p.KO) dst[c0 + jj + e] = __float2half_rn(__uint_as_float(r[jj + e]));
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (quarter == 0 && lane == 0) htrace_item(p, idx, 5);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  // A launch that did not wait for its predecessor before its work waits for it now, after its last
  // store: the kernel then cannot complete before everything queued ahead of it has, so completion
  // order along the stream stays transitive for whatever is queued next.
  if (p.independent) griddep_wait();
  if (threadIdx.x == 0 && p.trace != nullptr) {
    htrace(p, 3);
    p.trace[(size_t)blockIdx.x * kTraceWords + 4] = global_timer_ns();
  }
  if (warp == 3) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

struct HaloPlan {
  int Wp, TH, HR, RB, buf_bytes, box_bytes, b_stages;
  size_t smem;
};

bool plan(const ConvGeom& g, int bn, HaloPlan* out) {
  if (g.stride != 1 || (g.C % kBK) != 0 || g.R < 1 || g.S < 1 || g.R * g.S > 64 || g.Ho <= 0 || g.Wo <= 0) return false;
  const int Wp = g.W + 2 * g.pad;
  if (Wp > kBM || Wp > 256 || g.pad > 64) return false;
  const int TH = std::min(g.Ho, kBM / Wp);
  if (TH < 1) return false;
  const int HR = TH + g.R - 1;
  if (HR > 256) return false;
  const int rows_box = HR * Wp;
  const int rows_mma = kBM + (g.R - 1) * Wp + (g.S - 1);   // rows the last tap's window can reach
  const int rows = (std::max(rows_box, rows_mma) + 7) & ~7;
  const int buf_bytes = rows * 128;
  const size_t fixed = 1024 + (size_t)kHaloStages * 2 * buf_bytes + 256;
  const size_t budget = 227 * 1024;
  if (fixed + 3 * (size_t)bn * kBK * 2 > budget) return false;
  const int b_stages = (int)std::min<size_t>(kMaxBStages, (budget - fixed) / ((size_t)bn * kBK * 2));
  out->Wp = Wp; out->TH = TH; out->HR = HR; out->RB = (g.Ho + TH - 1) / TH;
  out->buf_bytes = buf_bytes; out->box_bytes = rows_box * 128; out->b_stages = b_stages;
  out->smem = fixed + (size_t)b_stages * bn * kBK * 2;
  return true;
}

template <int BN>
cudaError_t launch_halo(const CUtensorMap& tx, const CUtensorMap& tw, const HaloParams& p, int grid, size_t smem,
                        cudaStream_t stream) {
  auto kern = conv_f16_halo_kernel<BN>;
  static std::mutex mu;
  static size_t granted[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && granted[dev] < smem) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      granted[dev] = smem;
    }
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, tx, tw, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, smem, stream>>>(tx, tw, p);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace

// Tile widths the halo kernel is built for.
static int halo_tile_n(const helix_cfg_t* cfg, int KO) {
  if (cfg && cfg->tile_m != 0 && (cfg->tile_n == 64 || cfg->tile_n == 128)) return cfg->tile_n;
  return KO <= 64 ? 64 : 128;
}

bool conv_f16_halo_eligible(const ConvGeom& g, const helix_cfg_t* cfg) {
  HaloPlan pl;
  return encode_fn() != nullptr && plan(g, halo_tile_n(cfg, g.KO), &pl);
}

int conv_f16_halo_launch(const helix_cfg_t* cfg, const void* x, const void* w, void* y, const ConvGeom& g,
                         int* status_dev, int sm_count, bool independent, cudaStream_t stream, int64_t* launches) {
  const int bn = halo_tile_n(cfg, g.KO);
  HaloPlan pl;
  if (!plan(g, bn, &pl)) return HELIX_ERR_UNSUPPORTED;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return HELIX_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return HELIX_ERR_ALIGN;
  HaloParams p{};
  p.y = static_cast<__half*>(y);
  p.KO = g.KO; p.NB = g.NB; p.H = g.H; p.W = g.W; p.C = g.C; p.Ho = g.Ho; p.Wo = g.Wo; p.R = g.R; p.S = g.S; p.pad = g.pad;
  p.Wp = pl.Wp; p.TH = pl.TH; p.HR = pl.HR; p.RB = pl.RB;
  const int64_t blocks = (int64_t)g.NB * pl.RB;
  if (blocks <= 0 || blocks > 0x3fffffff) return HELIX_ERR_INVALID;
  p.blocks = (int)blocks;
  p.pairs = (p.blocks + 1) / 2;
  p.tiles_n = (g.KO + bn - 1) / bn;
  const int64_t items = (int64_t)p.pairs * p.tiles_n;
  if (items > 0x3fffffff) return HELIX_ERR_INVALID;
  p.items = (int)items;
  p.cblocks = g.C / kBK;
  p.taps = g.R * g.S;
  p.buf_bytes = pl.buf_bytes;
  p.box_bytes = pl.box_bytes;
  p.b_stages = pl.b_stages;
  p.independent = independent ? 1 : 0;
  p.vec_ok = ((g.KO & 7) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0) ? 1 : 0;
  p.status = status_dev;
  p.probe = (cfg && cfg->tile_m != 0) ? cfg->probe : 0;
  p.fd_tiles_n = make_fastdiv(p.tiles_n);
  p.fd_rb = make_fastdiv(p.RB);
  p.fd_wp = make_fastdiv(p.Wp);
  p.fd_s = make_fastdiv(p.S);

  CUtensorMap tx, tw;
  {
    // activations x[N][H][W][C] as a 4-D map (C, W, H, N); one box = 64 channels x Wp pixels x HR rows
    cuuint64_t dims[4] = {(cuuint64_t)g.C, (cuuint64_t)g.W, (cuuint64_t)g.H, (cuuint64_t)g.NB};
    cuuint64_t strides[3] = {(cuuint64_t)g.C * 2, (cuuint64_t)g.W * g.C * 2, (cuuint64_t)g.H * g.W * g.C * 2};
    cuuint32_t box[4] = {(cuuint32_t)kBK, (cuuint32_t)pl.Wp, (cuuint32_t)pl.HR, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (fn(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  {
    // weights w[KO][R*S*C] K-major; one box = 64 halves x bn rows
    const int64_t K = (int64_t)g.R * g.S * g.C;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)g.KO, 1};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)K * g.KO * 2};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)bn, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  const int grid = (int)std::min<int64_t>(items, sm_count);
  p.trace = gemm_f16_trace_for_grid(grid);
  const cudaError_t e = bn == 64 ? launch_halo<64>(tx, tw, p, grid, pl.smem, stream)
                                 : launch_halo<128>(tx, tw, p, grid, pl.smem, stream);
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  return HELIX_OK;
}

}  // namespace helix
