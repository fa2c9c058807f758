// Stride-2 NHWC convolution over 4 stored channels (an RGB network's first layer: 7 x 7, stride 2, pad 3, 3 + 1
// channels), with the input rows resident in shared memory and the im2col matrix never formed -- not in global
// memory (reference counterpart: src_template/Ampere_FP16/im2col.cu:37-97 writes the R*S-fold copy) and not in
// shared memory either.
//
// A pixel of 4 fp16 channels is 8 bytes, so two neighbouring pixels are one 16-byte K chunk and, with stride 2,
// the windows of neighbouring output pixels start 16 bytes apart.  That is exactly the canonical K-major layout of
// tcgen05.mma without swizzle -- row m of a core matrix at +16 m bytes -- with a LEADING byte offset of 16 as well:
// the operand "row ox, K chunk j" is the 16 bytes at  row_base + 16 (ox + j)  of the raw input row.  The matrix
// descriptor therefore reads the Toeplitz (overlapping-window) matrix straight from a raw image row; one filter row
// is K = 8 pixels x 4 channels = 32, two MMAs of 128 output pixels x KO x 16.  The window starts at pixel
// 2 ox - P with P = pad rounded up to even, so the filter's S taps sit at positions P - pad ... P - pad + S - 1 of
// the 8 (zero weights elsewhere).
//
// A work item is one output row (image b, row oy): 128 accumulator rows of which Wo <= 128 are stored.  Every CTA
// owns a contiguous strip of the (b, oy) list, so consecutive items share R - 2 of their R input rows; each input row
// is fetched once per strip with one untiled bulk copy (W * 8 contiguous bytes) into a ring of 16 row slots.  Zero
// padding left and right of the image is a zero margin of the row slot that no copy ever overwrites; filter rows that
// fall outside the image are skipped.  (A tiled TMA box of 16-byte pixel pairs would deliver the margins as
// out-of-bounds zeros, but its 16-byte inner extent makes it slower than the plain copies: 22.9 against 19.0 us.)
// The weights are rearranged once per CTA into the same unswizzled layout ([K chunk][KO / 8][8 x 16 bytes]).
//
// Roles (288 threads, two CTAs per SM): warp 0 row copies (lane k copies the item's k-th new row), warps 1-4 MMA
// issue (items round-robin, one accumulator per warp; convergent, one elected lane), warps 5-8 epilogue (TMEM -> fp16
// -> swizzled staging -> TMA store of full 128-byte lines).  All waits are bounded.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "conv_common.cuh"
#include "kernels.h"

namespace helix {

namespace {

constexpr int kBM = 128;             // output pixels per item (UMMA M)
constexpr int kThreads = 288;        // warp 0 row copies, warps 1-4 MMA issue, warps 5-8 epilogue
constexpr int kSlots = 16;           // input rows resident per CTA
constexpr int kPitch = 2176;         // bytes per row slot: margin + 256 pixels, and row 127's window (16 * 127 + 64)
constexpr int kRing = 16;            // items whose arrival / completion barriers are distinct
constexpr int kMaxR = 8;
constexpr int kPosPerRow = 8;        // window positions per filter row = K 32
constexpr int kChunksPerRow = 4;     // 16-byte K chunks per filter row
constexpr int kStagingBytes = 4 * 2 * 32 * 128;
constexpr int kTmemCols = 256;
constexpr int kBuildBarrier = 1;

struct StemParams {
  const uint8_t* x;     // [NB][H][W][4] fp16
  const uint8_t* w;     // [KO][R][S][4] fp16
  __half* y;            // [NB][Ho][Wo][KO]
  int NB, H, W, KO, R, S, pad, Ho, Wo;
  int P;                // zero margin left of pixel 0, in pixels (pad rounded up to even)
  int row_bytes;        // W * 8
  int items;            // NB * Ho
  int independent;
  int probe;            // tuning instrument: bit 0 = no MMAs, bit 1 = no row copies, bit 2 = no output stores
  int* status;
  FastDiv fd_ho;
  unsigned long long* trace;   // optional per-CTA stamps (null = off): words 0 / 4 global timer at start / end, 1-3 clock at start, after set-up, at the end
};

// Unswizzled K-major operand: 8-row groups `sbo` bytes apart, 16-byte K chunks `lbo` bytes apart.
// Bits: [0,14) address >> 4, [16,30) LBO >> 4, [32,46) SBO >> 4, [46,48) version = 1, [61,64) layout = 0.
__device__ __forceinline__ uint64_t umma_desc_plain(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(lbo >> 4) << 16;
  d |= static_cast<uint64_t>(sbo >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// The input rows an item needs and which of them are new.  Rows of one image segment occupy consecutive slots:
// slot(iy) = (seg_base + iy - seg_first) % kSlots.  Walked by the copying warp, which publishes the slot of each
// item's first row for the issuing warps.
struct RowWalk {
  int seg_base, seg_first, prev_hi, count;
  int lo, hi, new_lo;   // rows of the current item, first row to fetch (new_lo > hi: none)
  __device__ __forceinline__ void start() { seg_base = seg_first = count = 0; prev_hi = -1; }
  __device__ __forceinline__ void item(const StemParams& p, int first_of_strip, int oy) {
    lo = max(0, 2 * oy - p.pad);
    hi = min(p.H - 1, 2 * oy - p.pad + p.R - 1);
    if (first_of_strip || oy == 0) {
      seg_base = count;
      seg_first = lo;
      new_lo = lo;
    } else {
      new_lo = prev_hi + 1;
    }
    if (hi >= new_lo) count += hi - new_lo + 1;
    prev_hi = hi;   // never decreases inside an image
  }
  __device__ __forceinline__ int index_of(int iy) const { return seg_base + iy - seg_first; }
};

__device__ __forceinline__ void tr(const StemParams& p, int word, unsigned long long v) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * kTraceWords + word] = v;
}

// NACC accumulators of 256 / NACC columns each, one issuing warp per accumulator.  A single warp needs ~2400 cycles
// per item (14 MMAs handed over at ~60 cycles each, two barrier reads that queue behind them, its own scalar code at
// full instruction latency) against 448 cycles of tensor-pipe time, and the hand-over of an accumulator to the
// epilogue and back takes about a microsecond: items are independent, so they simply go round-robin to the warps.
template <int NACC>
__global__ void __launch_bounds__(kThreads, 2)
conv_f16_stem_kernel(const __grid_constant__ CUtensorMap tmap_y, const StemParams p) {
  griddep_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sOut = smem;                                          // [4 warps][2 boxes][32 pixels x 128 bytes], swizzled
  uint8_t* sRows = sOut + kStagingBytes;                         // [kSlots][kPitch]
  uint8_t* sB = sRows + (size_t)kSlots * kPitch;                 // [R * 4][KO / 8][128]
  const int b_bytes = p.R * kChunksPerRow * (p.KO / 8) * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + b_bytes);
  uint64_t* full = bars;                 // [kRing] rows of item i have landed
  uint64_t* done = bars + kRing;         // [kRing] MMAs of item i have completed
  uint64_t* tfull = bars + 2 * kRing;    // [4]
  uint64_t* tempty = bars + 2 * kRing + 4;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 2 * kRing + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* slot0_tab = reinterpret_cast<volatile int*>(tmem_ptr_smem + 2);   // [kRing] slot of item i's first row

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // this CTA's strip of the (image, output row) list
  const int t0 = (int)((int64_t)p.items * blockIdx.x / gridDim.x);
  const int t1 = (int)((int64_t)p.items * (blockIdx.x + 1) / gridDim.x);

  if (threadIdx.x == 0) {
    tr(p, 0, global_timer_ns());
    tr(p, 1, clock64());
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], 1);
    }
    for (int a = 0; a < NACC; ++a) {
      mbar_init(&tfull[a], 1);
      mbar_init(&tempty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_y);
  }
  // the margins of the row slots are the convolution's zero padding: written once, never touched by a copy
  // (the pixels in between are left alone, so that the first copies may land while this is still going on)
  {
    const int data0 = p.P * 8, data1 = p.P * 8 + p.row_bytes;
    for (int i = threadIdx.x; i < kSlots * (kPitch / 16); i += kThreads) {
      const int off = (i % (kPitch / 16)) * 16;
      if (off < data0 || off >= data1) reinterpret_cast<int4*>(sRows)[i] = make_int4(0, 0, 0, 0);
    }
  }
  if (warp == 1) tmem_alloc<kTmemCols>(tmem_ptr_smem);
  fence_proxy_async_smem();   // the zeros were written by ordinary stores, the tensor core reads them
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  if (!p.independent) griddep_wait();

  if (warp != 0) {
    // weights -> [K chunk j = r * 4 + jj][KO / 8][8 rows x 16 bytes]; chunk jj of filter row r holds window
    // positions 2 jj and 2 jj + 1, position q being filter column q - (P - pad).  Done by the warps that do not
    // copy rows, while the first rows are on their way; all loads of a pass are issued before its first store
    // (a pass costs one trip to L2; the 7 x 7 x 64 filter bank is one pass).
    constexpr int kBuilders = kThreads - 32, kBatch = 8;
    const int groups = p.KO / 8;
    const int ko_shift = p.KO == 64 ? 6 : 7;
    const int chunks = p.R * kChunksPerRow * p.KO;
    const int shift = p.P - p.pad;
    for (int c0 = threadIdx.x - 32; c0 < chunks; c0 += kBatch * kBuilders) {
      uint2 v[kBatch][2];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int c = c0 + u * kBuilders;
        const int n = c & (p.KO - 1), j = c >> ko_shift;
        const int r = j >> 2, jj = j & 3;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int s = 2 * jj + h - shift;
          v[u][h] = (c < chunks && s >= 0 && s < p.S)
                        ? __ldg(reinterpret_cast<const uint2*>(p.w + ((size_t)(n * p.R + r) * p.S + s) * 8))
                        : make_uint2(0u, 0u);
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int c = c0 + u * kBuilders;
        const int n = c & (p.KO - 1), j = c >> ko_shift;
        if (c < chunks)
          *reinterpret_cast<uint4*>(sB + ((size_t)j * groups + (n >> 3)) * 128 + (n & 7) * 16) =
              make_uint4(v[u][0].x, v[u][0].y, v[u][1].x, v[u][1].y);
      }
    }
    fence_proxy_async_smem();
    named_bar_sync(kBuildBarrier, kBuilders);
    if (threadIdx.x == 32) tr(p, 2, clock64());
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ row copies (whole warp, convergent)
    // Lane k issues the copy of the item's k-th new row; lane s < 16 remembers which item reads the row in slot s
    // last.  A slot is rewritten only after that item has completed; completion barriers are waited for in item
    // order and never more than kRing / 2 items late, so a parity can not be mistaken for an older one.
    bool ok = true;
    RowWalk rw;
    rw.start();
    int my_last = -1;
    int waited = -1;          // items up to here are known to be complete
    int b, oy;
    fast_divmod(t0, p.fd_ho, b, oy);
    for (int t = t0; t < t1; ++t) {
      const int i = t - t0;
      rw.item(p, i == 0, oy);
      const int nnew = rw.hi - rw.new_lo + 1;
      const int slot_first = rw.index_of(rw.new_lo) & (kSlots - 1);
      const int my_slot = (slot_first + lane) & (kSlots - 1);
      const int old = __shfl_sync(0xffffffffu, my_last, my_slot);
      const int need = max(__reduce_max_sync(0xffffffffu, lane < nnew ? old : -1), i - kRing / 2);
      for (; ok && waited < need; ++waited)
        ok = __all_sync(0xffffffffu, mbar_wait(&done[(waited + 1) & (kRing - 1)], ((waited + 1) / kRing) & 1, abort_flag,
                                               p.status));
      if (!ok) break;
      uint64_t* const fb = &full[i & (kRing - 1)];
      if (lane == 0) slot0_tab[i & (kRing - 1)] = rw.index_of(rw.lo) & (kSlots - 1);   // published by the arrival
      if (nnew > 0 && !(p.probe & 2)) {
        if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)(nnew * p.row_bytes));
        __syncwarp();
        if (lane < nnew)
          bulk_load(sRows + (size_t)my_slot * kPitch + p.P * 8,
                    p.x + ((size_t)((int64_t)b * p.H + rw.new_lo + lane) * p.W) * 8, (uint32_t)p.row_bytes, fb);
      } else if (lane == 0) {
        mbar_arrive(fb);
      }
      // row iy is read last by output row (iy + pad) / 2 of this image, if the strip gets that far
      const int k = (lane - slot_first) & (kSlots - 1);
      if (lane < kSlots && k < nnew) my_last = i + min((rw.new_lo + k + p.pad) >> 1, p.Ho - 1) - oy;
      if (++oy == p.Ho) { oy = 0; ++b; }
    }
  } else if (warp <= 4) {
    // ------------------------------------------------------------------ MMA issue (whole warp, one elected lane)
    // Warp ME issues items ME, ME + NACC, ... into accumulator ME.  The descriptors are kept as 32-bit low words
    // that advance by additions (the high words are constants) and the filter rows are unrolled: a warp that runs
    // alone pays the full latency of every dependent instruction.
    const int ME = warp - 1;
    if (ME < NACC) {
      const uint32_t idesc = umma_idesc_f16(kBM, p.KO);
      const uint32_t lbo_b16 = (uint32_t)(p.KO / 8) * 8u;                     // K chunk stride of B, in 16-byte units
      // A: row ox at +16 ox (8-row groups 128 bytes apart), K chunks 16 bytes apart; B: groups 128 bytes, chunks lbo_b
      const uint32_t a_lo0 = ((smem_u32(sRows) & 0x3FFFF) >> 4) | (1u << 16);
      const uint32_t b_lo0 = ((smem_u32(sB) & 0x3FFFF) >> 4) | (lbo_b16 << 16);
      constexpr uint32_t kDescHi = (128u >> 4) | (1u << 14);                  // SBO = 128 bytes, version 1
      const uint32_t b_row_step = kChunksPerRow * lbo_b16, b_half_step = 2 * lbo_b16;
      const bool issue = !(p.probe & 1);
      const uint32_t d_tmem = tmem_base + ME * (kTmemCols / NACC);
      bool ok = true;
      int seen = -1;   // arrival barriers up to this item have been seen: an item also reads rows that came with its
                       // predecessors, whose barriers other warps wait for
      int b, oy;
      fast_divmod(t0 + ME, p.fd_ho, b, oy);
      for (int i = ME; ok && t0 + i < t1; i += NACC) {
        ok = __all_sync(0xffffffffu, mbar_wait(&tempty[ME], ((i / NACC) & 1) ^ 1, abort_flag, p.status));
        if (!ok) break;
        for (; ok && seen < i; ++seen)
          ok = __all_sync(0xffffffffu, mbar_wait(&full[(seen + 1) & (kRing - 1)], ((seen + 1) / kRing) & 1, abort_flag,
                                                 p.status));
        if (!ok) break;
        int slot = slot0_tab[i & (kRing - 1)];
        tc_fence_after_sync();
        const int r_lo = max(0, p.pad - 2 * oy), r_hi = min(p.R - 1, p.H - 1 + p.pad - 2 * oy);   // rows inside the image
#pragma unroll
        for (int r = 0; r < kMaxR; ++r) {
          if (r >= r_lo && r <= r_hi) {   // warp-uniform
            const uint32_t a_lo = a_lo0 + (uint32_t)slot * (kPitch / 16);
            const uint32_t b_lo = b_lo0 + (uint32_t)r * b_row_step;
            if (issue) {
              umma_f16_ss_elect(d_tmem, ((uint64_t)kDescHi << 32) | a_lo, ((uint64_t)kDescHi << 32) | b_lo, idesc,
                                r != r_lo);
              umma_f16_ss_elect(d_tmem, ((uint64_t)kDescHi << 32) | (a_lo + 2),
                                ((uint64_t)kDescHi << 32) | (b_lo + b_half_step), idesc, true);
            }
            slot = (slot + 1) & (kSlots - 1);
          }
        }
        umma_commit_elect(&done[i & (kRing - 1)]);
        umma_commit_elect(&tfull[ME]);
        oy += NACC;
        while (oy >= p.Ho) oy -= p.Ho;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    // TMEM lane = output pixel ox of the row, column = output channel.  64 channels at a time go TMEM -> registers
    // -> fp16 -> this warp's swizzled 32 x 128-byte staging box -> one TMA store (full lines; pixels beyond Wo are
    // clipped by the tensor map).  Two boxes per warp alternate, so one is filled while the other drains; the
    // accumulator is handed back as soon as it is in registers.
    const int quarter = warp & 3;
    uint8_t* const boxes = sOut + (size_t)quarter * (2 * 32 * 128);
    int box = 0;
    bool ok = true;
    for (int t = t0; ok && t < t1; ++t) {
      const int i = t - t0;
      const int acc = i % NACC;
      ok = mbar_wait(&tfull[acc], (i / NACC) & 1, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * (kTmemCols / NACC);
      for (int c0 = 0; c0 < p.KO; c0 += 64) {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32b_x32(taddr + c0, lo);
        tmem_ld_32x32b_x32(taddr + c0 + 32, hi);
        tmem_ld_wait();
        if (c0 + 64 >= p.KO) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty[acc]);
        }
        if (quarter * 32 >= p.Wo || (p.probe & 4)) continue;   // warp-uniform: nothing of this warp's is stored
        uint8_t* const stage_box = boxes + box * (32 * 128);
        const uint32_t row_base = smem_u32(stage_box) + lane * 128;
        box ^= 1;
        if (lane == 0) tma_store_wait_read_1();   // the store issued two boxes ago has left this buffer
        __syncwarp();
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint32_t* src = ch < 4 ? &lo[ch * 8] : &hi[(ch - 4) * 8];
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((ch ^ (lane & 7)) << 4)),
                       "r"(pack_half2(__uint_as_float(src[0]), __uint_as_float(src[1]))),
                       "r"(pack_half2(__uint_as_float(src[2]), __uint_as_float(src[3]))),
                       "r"(pack_half2(__uint_as_float(src[4]), __uint_as_float(src[5]))),
                       "r"(pack_half2(__uint_as_float(src[6]), __uint_as_float(src[7])))
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&tmap_y, stage_box, c0, quarter * 32, t);
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait_all();   // nothing of this thread's is in flight when the CTA tears down
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  // a launch that did not wait for its predecessor before its work waits for it now, so that completion order
  // along the stream stays transitive
  if (p.independent) griddep_wait();
  if (threadIdx.x == 0) {
    tr(p, 3, clock64());
    tr(p, 4, global_timer_ns());
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

size_t stem_smem_bytes(const ConvGeom& g) {
  return 1024 + kStagingBytes + (size_t)kSlots * kPitch + (size_t)g.R * kChunksPerRow * (g.KO / 8) * 128 + (2 * kRing + 8) * 8 + 16 + kRing * 4;
}

}  // namespace

bool conv_f16_stem_eligible(const ConvGeom& g) {
  if (g.C != 4 || g.stride != 2 || g.R < 2 || g.R > kMaxR || g.S < 1 || g.pad < 0 || g.pad >= g.R) return false;
  const int P = (g.pad + 1) & ~1;
  if (P - g.pad + g.S > kPosPerRow) return false;                      // the taps fit the 8 window positions
  if (g.Wo < 1 || g.Wo > kBM || g.Ho < 1 || (g.W & 1)) return false;   // one item = one output row; rows of 16 n bytes
  if ((P + g.W) * 8 > kPitch) return false;
  if (g.KO != 64 && g.KO != 128) return false;                        // whole 128-byte staging rows
  return (int64_t)g.NB * g.Ho <= 0x3fffffff;
}

int conv_f16_stem_launch(const void* x, const void* w, void* y, const ConvGeom& g, int probe, int* status_dev,
                         int sm_count, bool independent, cudaStream_t stream, int64_t* launches) {
  if (!conv_f16_stem_eligible(g)) return HELIX_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(y) & 15))
    return HELIX_ERR_ALIGN;
  StemParams p{};
  p.x = static_cast<const uint8_t*>(x);
  p.w = static_cast<const uint8_t*>(w);
  p.y = static_cast<__half*>(y);
  p.NB = g.NB; p.H = g.H; p.W = g.W; p.KO = g.KO; p.R = g.R; p.S = g.S; p.pad = g.pad; p.Ho = g.Ho; p.Wo = g.Wo;
  p.P = (g.pad + 1) & ~1;
  p.row_bytes = g.W * 8;
  p.items = g.NB * g.Ho;
  p.independent = independent ? 1 : 0;
  p.probe = probe;
  p.status = status_dev;
  p.fd_ho = make_fastdiv(g.Ho);
  // y[NB][Ho][Wo][KO] as (KO, Wo, NB * Ho); one box = 64 channels x 32 pixels of one output row
  EncodeTiledFn fn = conv_tensor_map_encoder();
  if (!fn) return HELIX_ERR_CUDA;
  CUtensorMap ty;
  {
    cuuint64_t dims[3] = {(cuuint64_t)g.KO, (cuuint64_t)g.Wo, (cuuint64_t)p.items};
    cuuint64_t strides[2] = {(cuuint64_t)g.KO * 2, (cuuint64_t)g.Wo * g.KO * 2};
    cuuint32_t box[3] = {64, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&ty, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return HELIX_ERR_CUDA;
  }
  const size_t smem = stem_smem_bytes(g);
  const bool narrow = g.KO <= 64;
  auto kern = narrow ? conv_f16_stem_kernel<4> : conv_f16_stem_kernel<2>;
  {
    static std::mutex mu;
    static size_t granted[2][64] = {{0}};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && granted[narrow][dev] < smem) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return HELIX_ERR_CUDA;
      granted[narrow][dev] = smem;
    }
  }
  // two CTAs per SM: one's epilogue and set-up run under the other's MMAs
  const int grid = (int)std::min<int64_t>(p.items, 2 * (int64_t)sm_count);
  p.trace = gemm_f16_trace_for_grid(grid);
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
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, ty, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, smem, stream>>>(ty, p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  return HELIX_OK;
}

}  // namespace helix
