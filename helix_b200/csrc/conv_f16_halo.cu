// Stride-1 NHWC convolution with the input window resident in shared memory ("window" variant).
//
// The implicit-GEMM kernel in gemm_f16_tc.cu fetches every input pixel once per filter tap (R*S times)
// through the im2col tensor map and is bound by that operand traffic from L2 (reference counterpart:
// src_template/Ampere_FP16/im2col.cu:37-97 materialises the R*S-fold copy in global memory).  Here a work
// item is a block of TH whole output rows of one image times a tile of 128 output channels:
//   * its input window -- TH + R - 1 padded rows of Wp = W + 2*pad pixels, 64 channels -- is brought in by
//     ONE tiled TMA box per channel block (out-of-image pixels arrive as zeros) and laid out as rows of 128
//     bytes, row index q = h*Wp + w, 128-byte swizzled;
//   * the GEMM N axis runs over the padded positions q = hl*Wp + wl of the block (up to 256; positions with
//     wl >= Wo are junk columns that are never stored), so the B operand of filter tap (r, s) is the SAME
//     buffer read from row r*Wp + s on: the tap only moves the start address of the matrix descriptor;
//   * the output channels sit on the 128-row M axis (a tcgen05.mma costs its issuing thread about the same
//     whatever its width, so the wide axis belongs to the pixels): the A operand is a 128 x 64 slab of the
//     weights per tap and channel block, streamed through a ring;
//   * the accumulator (128 channels x up to 256 positions, fp32) lives in TMEM, double buffered;
//   * the epilogue writes 2 bytes per lane: the 32 lanes of a warp are 32 consecutive output channels of
//     one pixel, i.e. 64 contiguous bytes of y.
// Each input byte is loaded once per item instead of R*S times.
//
// Roles (384 threads): warp 0 window loads, warps 1-2 weight-slab loads (alternating slabs), warp 3 MMA
// issue + TMEM allocation, warps 4-11 epilogue (two warps per quarter of the TMEM lanes, alternate 32-column
// chunks).  The weight ring's arrival barriers are shared by groups of slabs so that the issuing thread
// reads one barrier per group.  All waits are bounded.
//
// Measured on B200 (32 images): the kernel is level with the im2col path at 128 channels / 28x28 and behind it
// where the tile shape fits badly (64 output channels use half of the 128 accumulator rows; a 7x7 image fills a
// quarter of the 256 columns), so it is an explicit variant (conv_gather = 3), not a default.
#include <cuda.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "conv_common.cuh"
#include "kernels.h"

namespace helix {

namespace {

constexpr int kBM = 128;          // output channels per tile (UMMA M)
constexpr int kBK = 64;
constexpr int kMaxPos = 256;      // padded positions per block (UMMA N)
constexpr int kThreads = 384;
constexpr int kWinStages = 2;     // windows in flight
constexpr int kMaxWStages = 8;    // weight-slab ring
constexpr int kWBytes = kBM * kBK * 2;
constexpr int kWWarps = 2;
constexpr int kTmemCols = 2 * kMaxPos;

struct WinParams {
  __half* y;
  int KO, NB, H, W, C, Ho, Wo, R, S, pad;
  int Wp;            // padded row length = W + 2 * pad
  int TH;            // output rows per block, TH * Wp <= 256
  int HR;            // input rows per block = TH + R - 1
  int RB;            // row blocks per image
  int blocks;        // NB * RB
  int tiles_m;       // output-channel tiles of 128
  int items;         // blocks * tiles_m
  int cblocks;       // C / 64
  int taps;          // R * S
  int npos;          // UMMA N: TH * Wp rounded up to 16
  int buf_bytes;     // bytes of one window buffer (multiple of 1024)
  int box_bytes;     // bytes one window box delivers = HR * Wp * 128
  int w_stages;
  int w_group;       // weight slabs per arrival barrier (divides w_stages): the MMA issuer waits once per group
  int independent;
  int probe;         // tuning instrument (helix_cfg_t.probe): 1 = issue no MMA
  int* status;
  FastDiv fd_tiles_m, fd_rb, fd_wp, fd_wgroup;
  unsigned long long* trace;   // optional per-CTA timeline (null = off), same layout as the GEMM kernels
};

__device__ __forceinline__ void wtrace(const WinParams& p, int word) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * kTraceWords + word] = (unsigned long long)clock64();
}
__device__ __forceinline__ void wtrace_item(const WinParams& p, int idx, int slot) {
  if (idx < kTraceTiles) wtrace(p, 8 + idx * 6 + slot);
}
__device__ __forceinline__ void wtrace_slab(const WinParams& p, int which, int n) {
  if (n < kTraceSlabs) wtrace(p, 8 + 6 * kTraceTiles + which * kTraceSlabs + n);
}

struct WinItem {
  int mb;            // output-channel tile
  int img, ho0;      // image and first output row of the block
};

// Items of one block (all its channel tiles) are consecutive, so that the CTAs working on them share
// the window in L2.
__device__ __forceinline__ bool win_item(const WinParams& p, int t, WinItem& it) {
  if (t >= p.items) return false;
  int blk, rb;
  fast_divmod(t, p.fd_tiles_m, blk, it.mb);
  fast_divmod(blk, p.fd_rb, it.img, rb);
  it.ho0 = rb * p.TH;
  return true;
}

// Slab n of the CTA's sequence belongs to issuer n % nissue: the first tap of `issuer` inside a run of taps whose
// first slab has sequence number `first`.
__device__ __forceinline__ int issuer_first_tap(int first, int nissue, int issuer) {
  const int r = first % nissue;
  return issuer >= r ? issuer - r : issuer - r + nissue;
}

__global__ void __launch_bounds__(kThreads, 1)
conv_f16_win_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const WinParams p) {
  griddep_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sWin = smem;                                              // [kWinStages][buf_bytes]
  uint8_t* sW = smem + (size_t)kWinStages * p.buf_bytes;            // [w_stages][kWBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sW + (size_t)p.w_stages * kWBytes);
  uint64_t* hfull = bars;            // [2]
  uint64_t* hempty = bars + 2;       // [2]
  uint64_t* wfull = bars + 4;        // [8]
  uint64_t* wempty = bars + 12;      // [8]
  uint64_t* tfull = bars + 20;       // [2]
  uint64_t* tempty = bars + 22;      // [2]
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 24);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  int* off_tab = reinterpret_cast<int*>(bars + 26);   // [kMaxPos]: element offset of each position in y, or -1

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = blockIdx.x;
  const int grid = gridDim.x;

  if (threadIdx.x == 0) {
    if (p.trace != nullptr) {
      p.trace[(size_t)blockIdx.x * kTraceWords + 0] = global_timer_ns();
      wtrace(p, 1);
    }
    for (int s = 0; s < kWinStages; ++s) {
      mbar_init(&hfull[s], 1);
      mbar_init(&hempty[s], 1);
    }
    for (int s = 0; s < p.w_stages; ++s) {
      if (s * p.w_group < p.w_stages) mbar_init(&wfull[s], p.w_group);
      mbar_init(&wempty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], kThreads / 32 - 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
  }
  // Where each padded position q = hl * Wp + wl of a block lands in y relative to the block's first pixel
  // (channel 0), or -1 for the junk positions wl >= Wo: the same for every item, so decoded once.
  for (int q = threadIdx.x; q < kMaxPos; q += blockDim.x) {
    int hl, wl;
    fast_divmod(q, p.fd_wp, hl, wl);
    off_tab[q] = (wl < p.Wo && hl < p.TH) ? (hl * p.Wo + wl) * p.KO : -1;
  }
  if (warp == 3) tmem_alloc<kTmemCols>(tmem_ptr_smem);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (!p.independent) griddep_wait();
  if (threadIdx.x == 0) wtrace(p, 2);

  if (warp == 0) {
    // ------------------------------------------------------------------ window loads
    if (lane == 0) {
      bool ok = true;
      int hs = 0;          // window ring stage and its use parity
      uint32_t ph = 0;
      WinItem it;
      int idx = 0;
      for (int t = cta; ok && win_item(p, t, it); t += grid, ++idx) {
        for (int cb = 0; cb < p.cblocks && ok; ++cb) {
          ok = mbar_wait(&hempty[hs], ph ^ 1, abort_flag, p.status);
          if (!ok) break;
          wtrace_item(p, idx, cb == 0 ? 0 : 1);
          mbar_arrive_expect_tx(&hfull[hs], (uint32_t)p.box_bytes);
          tma_load_4d(sWin + (size_t)hs * p.buf_bytes, &tmap_x, &hfull[hs], cb * kBK, -p.pad, it.ho0 - p.pad, it.img);
          if (++hs == kWinStages) { hs = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp <= kWWarps) {
    // ------------------------------------------------------------------ weight-slab loads
    // slab sequence: for each item, for each channel block, for each tap; slab n belongs to issuer
    // n % kWWarps (an issuing thread is held a few hundred cycles per tensor copy)
    const int issuer = warp - 1;
    const int nissue = min(kWWarps, p.w_stages);
    if (lane == 0 && issuer < nissue) {
      bool ok = true;
      int ws = issuer;          // ring stage of this issuer's next slab, its use parity, its group's barrier
      uint32_t ph = 0;
      int total = 0;            // slabs of the whole CTA (all issuers), for the padding of the last group
      WinItem it;
      for (int t = cta; ok && win_item(p, t, it); t += grid) {
        for (int cb = 0; cb < p.cblocks && ok; ++cb) {
          for (int tap = issuer_first_tap(total, nissue, issuer); tap < p.taps; tap += nissue) {
            ok = mbar_wait(&wempty[ws], ph ^ 1, abort_flag, p.status);
            if (!ok) break;
            wtrace_slab(p, 0, total + tap);
            uint64_t* const fb = &wfull[fast_div(ws, p.fd_wgroup)];
            mbar_arrive_expect_tx(fb, kWBytes);
            // rows beyond KO (a last, ragged channel tile) arrive as zeros
            tma_load_3d(sW + (size_t)ws * kWBytes, &tmap_w, fb, tap * p.C + cb * kBK, it.mb * kBM, 0);
            ws += nissue;
            if (ws >= p.w_stages) { ws -= p.w_stages; ph ^= 1; }
          }
          total += p.taps;
        }
      }
      // a short last group of the CTA's slab sequence is completed by plain arrivals, each ordered after the
      // release of its ring stage like a real slab
      const int padded = (total + p.w_group - 1) / p.w_group * p.w_group;
      for (int n = total + ((issuer - total % nissue) + nissue) % nissue; ok && n < padded; n += nissue) {
        ok = mbar_wait(&wempty[ws], ph ^ 1, abort_flag, p.status);
        if (!ok) break;
        mbar_arrive(&wfull[fast_div(ws, p.fd_wgroup)]);
        ws += nissue;
        if (ws >= p.w_stages) { ws -= p.w_stages; ph ^= 1; }
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ MMA issuer
    // the whole warp walks the loop convergently (warp-uniform state, waits end in a vote); one elected lane issues
    {
      const uint32_t idesc = umma_idesc_f16(kBM, p.npos);
      bool ok = true;
      int idx = 0, nslab = 0;
      int hs = 0, ws = 0, gpos = 0, gidx = 0;     // window stage; weight stage, position in its group, group
      uint32_t hph = 0, wph = 0;
      WinItem it;
      for (int t = cta; ok && win_item(p, t, it); t += grid, ++idx) {
        const int acc = idx & 1;
        const uint32_t acc_phase = (idx >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&tempty[acc], acc_phase ^ 1, abort_flag, p.status));
        if (!ok) break;
        tc_fence_after_sync();
        if (lane == 0) wtrace_item(p, idx, 2);
        const uint32_t d_tmem = tmem_base + acc * kMaxPos;
        for (int cb = 0; cb < p.cblocks && ok; ++cb) {
          ok = __all_sync(0xffffffffu, mbar_wait(&hfull[hs], hph, abort_flag, p.status));
          if (!ok) break;
          const uint32_t win0 = smem_u32(sWin + (size_t)hs * p.buf_bytes);
          uint32_t tap_row = 0;      // first window row of the tap, in bytes: (fr * Wp + fs) * 128
          int fs = 0;
          for (int tap = 0; tap < p.taps; ++tap) {
            // one wait per group of weight slabs: reading the barrier costs this thread some 200 cycles on
            // top of the 45 it needs to hand an MMA to the tensor core; the stages are released one by one
            if (gpos == 0) {
              ok = __all_sync(0xffffffffu, mbar_wait(&wfull[gidx], wph, abort_flag, p.status));
              if (!ok) break;
            }
            if (++gpos == p.w_group) { gpos = 0; ++gidx; }
            if (lane == 0) wtrace_slab(p, 1, nslab);
            ++nslab;
            tc_fence_after_sync();
            const uint64_t da = umma_desc_sw128(smem_u32(sW + (size_t)ws * kWBytes));
            // The tensor core derives the swizzle phase of a row from the row's absolute shared-memory
            // address, exactly as the TMA did when it wrote the rows, so a window that starts at any row
            // is described by its plain start address.
            const uint64_t db = umma_desc_sw128(win0 + tap_row);
            if (!(p.probe & 1)) {
#pragma unroll
              for (int k = 0; k < kBK / 16; ++k)
                umma_f16_ss_elect(d_tmem, da + 2 * k, db + 2 * k, idesc, (cb > 0) || (tap > 0) || (k > 0));
            }
            umma_commit_elect(&wempty[ws]);
            if (++ws == p.w_stages) { ws = 0; wph ^= 1; gidx = 0; }
            tap_row += 128u;
            if (++fs == p.S) { fs = 0; tap_row += (uint32_t)(p.Wp - p.S) * 128u; }
          }
          if (ok) umma_commit_elect(&hempty[hs]);
          if (++hs == kWinStages) { hs = 0; hph ^= 1; }
        }
        if (ok) umma_commit_elect(&tfull[acc]);
        if (lane == 0) wtrace_item(p, idx, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // TMEM lane = output channel of the tile, column = padded position of the block.  For one column
    // the 32 lanes of a warp are 32 consecutive channels of one pixel: 64 contiguous bytes of y.
    // Two warps share each quarter of the lanes and take alternate 32-column chunks.
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    bool ok = true;
    int idx = 0;
    WinItem it;
    for (int t = cta; ok && win_item(p, t, it); t += grid, ++idx) {
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      ok = mbar_wait(&tfull[acc], acc_phase, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      if (warp == 4 && lane == 0) wtrace_item(p, idx, 4);
      const int ko = it.mb * kBM + quarter * 32 + lane;
      // Offsets below `limit` are pixels of output rows inside the image; the junk positions carry -1, which
      // as an unsigned number is above every limit, and a channel beyond KO gets the limit 0.
      const int rows_left = min(p.TH, p.Ho - it.ho0);
      const uint32_t limit = ko < p.KO ? (uint32_t)(rows_left * p.Wo * p.KO) : 0u;
      __half* const ybase = p.y + ((int64_t)it.img * p.Ho + it.ho0) * p.Wo * p.KO + ko;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kMaxPos + half * 32;
      const int* const tab = off_tab + half * 32;
      const int nmine = (p.npos - half * 32 + 63) >> 6;     // this warp's chunks: columns half*32 + 64*i
      uint32_t r0[32], r1[32];
      auto put = [&](const uint32_t (&r)[32], int c0) {
#pragma unroll
        for (int j4 = 0; j4 < 32; j4 += 4) {
          const int4 o = *reinterpret_cast<const int4*>(tab + c0 + j4);
          if ((uint32_t)o.x < limit) ybase[o.x] = __float2half_rn(__uint_as_float(r[j4 + 0]));
          if ((uint32_t)o.y < limit) ybase[o.y] = __float2half_rn(__uint_as_float(r[j4 + 1]));
          if ((uint32_t)o.z < limit) ybase[o.z] = __float2half_rn(__uint_as_float(r[j4 + 2]));
          if ((uint32_t)o.w < limit) ybase[o.w] = __float2half_rn(__uint_as_float(r[j4 + 3]));
        }
      };
      if (nmine > 0) tmem_ld_32x32b_x32(taddr, r0);
#pragma unroll
      for (int i = 0; i < kMaxPos / 64; i += 2) {
        if (i < nmine) {       // uniform over the warp
          tmem_ld_wait();
          if (i + 1 < nmine) tmem_ld_32x32b_x32(taddr + (i + 1) * 64, r1);
          put(r0, i * 64);
          if (i + 1 < nmine) {
            tmem_ld_wait();
            if (i + 2 < nmine) tmem_ld_32x32b_x32(taddr + (i + 2) * 64, r0);
            put(r1, (i + 1) * 64);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (warp == 4 && lane == 0) wtrace_item(p, idx, 5);
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
    wtrace(p, 3);
    p.trace[(size_t)blockIdx.x * kTraceWords + 4] = global_timer_ns();
  }
  if (warp == 3) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

struct WinPlan {
  int Wp, TH, HR, RB, npos, buf_bytes, box_bytes, w_stages;
  size_t smem;
};

bool plan(const ConvGeom& g, WinPlan* out) {
  if (g.stride != 1 || (g.C % kBK) != 0 || g.R < 1 || g.S < 1 || g.R * g.S > 64 || g.Ho <= 0 || g.Wo <= 0) return false;
  const int Wp = g.W + 2 * g.pad;
  if (Wp > kMaxPos || Wp < 2 || g.pad > 64) return false;
  const int TH = std::min(g.Ho, kMaxPos / Wp);
  if (TH < 1) return false;
  const int HR = TH + g.R - 1;
  if (HR > 256) return false;
  const int npos = (TH * Wp + 15) & ~15;
  const int rows_box = HR * Wp;
  const int rows_mma = npos + (g.R - 1) * Wp + (g.S - 1);   // rows the last tap's window can reach
  const int rows = (std::max(rows_box, rows_mma) + 7) & ~7;
  const int buf_bytes = rows * 128;
  const size_t fixed = 1024 + (size_t)kWinStages * buf_bytes + 256 + kMaxPos * sizeof(int);
  const size_t budget = 227 * 1024;
  if (fixed + 3 * (size_t)kWBytes > budget) return false;
  const int w_stages = (int)std::min<size_t>(kMaxWStages, (budget - fixed) / kWBytes);
  out->Wp = Wp; out->TH = TH; out->HR = HR; out->RB = (g.Ho + TH - 1) / TH; out->npos = npos;
  out->buf_bytes = buf_bytes; out->box_bytes = rows_box * 128; out->w_stages = w_stages;
  out->smem = fixed + (size_t)w_stages * kWBytes;
  return true;
}

}  // namespace

EncodeTiledFn conv_tensor_map_encoder() {
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

bool conv_f16_halo_eligible(const ConvGeom& g, const helix_cfg_t* cfg) {
  (void)cfg;
  WinPlan pl;
  return conv_tensor_map_encoder() != nullptr && plan(g, &pl);
}

// Microseconds the window kernel is expected to take, or a negative value when the geometry is not covered:
// rounds of items over the SMs times the time of an item (an MMA of 128 x N x 16 takes N / 2 cycles, but the
// issuing thread was measured at no less than ~580 cycles per tap of four), plus launch and the last epilogue.
double conv_f16_halo_estimate_us(const ConvGeom& g, int sm_count) {
  WinPlan pl;
  if (!conv_f16_halo_eligible(g, nullptr) || !plan(g, &pl)) return -1.0;
  const int64_t items = (int64_t)g.NB * pl.RB * ((g.KO + kBM - 1) / kBM);
  const int64_t rounds = (items + sm_count - 1) / sm_count;
  const double tap_cycles = std::max(580.0, 4.0 * pl.npos / 2.0 * 1.25);
  const double item_us = (double)(g.C / kBK) * g.R * g.S * tap_cycles / 1750.0;
  return rounds * item_us + 3.3 + 2.0;
}

int conv_f16_halo_launch(const helix_cfg_t* cfg, const void* x, const void* w, void* y, const ConvGeom& g,
                         int* status_dev, int sm_count, bool independent, cudaStream_t stream, int64_t* launches) {
  WinPlan pl;
  if (!plan(g, &pl)) return HELIX_ERR_UNSUPPORTED;
  EncodeTiledFn fn = conv_tensor_map_encoder();
  if (!fn) return HELIX_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return HELIX_ERR_ALIGN;
  WinParams p{};
  p.y = static_cast<__half*>(y);
  p.KO = g.KO; p.NB = g.NB; p.H = g.H; p.W = g.W; p.C = g.C; p.Ho = g.Ho; p.Wo = g.Wo; p.R = g.R; p.S = g.S; p.pad = g.pad;
  p.Wp = pl.Wp; p.TH = pl.TH; p.HR = pl.HR; p.RB = pl.RB; p.npos = pl.npos;
  const int64_t blocks = (int64_t)g.NB * pl.RB;
  if (blocks <= 0 || blocks > 0x3fffffff) return HELIX_ERR_INVALID;
  p.blocks = (int)blocks;
  p.tiles_m = (g.KO + kBM - 1) / kBM;
  const int64_t items = blocks * p.tiles_m;
  if (items > 0x3fffffff) return HELIX_ERR_INVALID;
  p.items = (int)items;
  p.cblocks = g.C / kBK;
  p.taps = g.R * g.S;
  p.buf_bytes = pl.buf_bytes;
  p.box_bytes = pl.box_bytes;
  // weight slabs per arrival barrier: a filter row where that divides the ring, else 2 (or 1)
  p.w_group = (g.S <= 4 && pl.w_stages >= 2 * g.S) ? g.S : (pl.w_stages >= 4 ? 2 : 1);
  if ((cfg->probe >> 4) & 7) p.w_group = min((cfg->probe >> 4) & 7, pl.w_stages);
  p.w_stages = pl.w_stages / p.w_group * p.w_group;
  p.fd_wgroup = make_fastdiv(p.w_group);
  p.independent = independent ? 1 : 0;
  p.status = status_dev;
  p.probe = (cfg && cfg->tile_m != 0) ? (cfg->probe & 1) : 0;
  p.fd_tiles_m = make_fastdiv(p.tiles_m);
  p.fd_rb = make_fastdiv(p.RB);
  p.fd_wp = make_fastdiv(p.Wp);

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
    // weights w[KO][R*S*C] K-major; one box = 64 halves x 128 output channels
    const int64_t K = (int64_t)g.R * g.S * g.C;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)g.KO, 1};
    cuuint64_t strides[2] = {(cuuint64_t)K * 2, (cuuint64_t)K * g.KO * 2};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)kBM, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(w), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  const int grid = (int)std::min<int64_t>(items, sm_count);
  p.trace = gemm_f16_trace_for_grid(grid);
  auto kern = conv_f16_win_kernel;
  {
    static std::mutex mu;
    static size_t granted[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && granted[dev] < pl.smem) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) != cudaSuccess)
        return HELIX_ERR_CUDA;
      granted[dev] = pl.smem;
    }
  }
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(grid);
  lc.blockDim = dim3(kThreads);
  lc.dynamicSmemBytes = pl.smem;
  lc.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = attr;
  lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, tx, tw, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, pl.smem, stream>>>(tx, tw, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  return HELIX_OK;
}

}  // namespace helix
