// fp16 GEMM and implicit-GEMM NHWC convolution on the sm_100a tensor cores.
//
//   D[PM, PN] (fp32 in TMEM) = OpA[PM, K] * OpB[PN, K]^T      both operands K-major fp16
//
// Counterpart of the reference's mmaPermuted_Coalesced_32Stride (src_template/Ampere_FP16/gemm.cu
// :120-534), its split-K twin (gemm_splitK.cu:120-509) and, for convolution, of the im2col +
// GEMM pair (src_template/Ampere_FP16/im2col.cu:37-75; scripts/Ampere_FP16/Ampere_FP16_conv.py
// :431-446).  Where the reference stages 32-wide K slabs with cp.async, feeds mma.sync from
// ldmatrix fragments and accumulates in fp16 registers, this kernel:
//   * moves 128 x 64 (A side) and BN x 64 (B side) fp16 tiles with TMA into a ring of
//     128B-swizzled shared-memory stages guarded by full/empty mbarriers;
//   * issues tcgen05.mma.kind::f16 (M = 128, N = BN, K = 16) from one thread, operands read
//     straight from shared memory through matrix descriptors, fp32 accumulators in TMEM;
//   * is persistent: each CTA walks a rasterised list of output tiles, and the accumulator is
//     double buffered in TMEM so the epilogue of tile i overlaps the main loop of tile i+1;
//   * epilogue warps read TMEM with tcgen05.ld, round once to fp16 and store to global memory
//     (or store fp32 partials for split-K, reduced in slice order by a second kernel);
//   * swap_ab puts the large N extent on the 128-row UMMA axis when M is skinny.
// For convolution the A-side tile is gathered by 128 producer threads with 16-byte zero-filling
// cp.async (8 lanes per output pixel, K axis ordered (r, s, c)), written in the same swizzled
// layout the TMA would produce; each thread's arrival on the stage barrier fires when its copies
// land, and the MMA thread issues fence.proxy.async before the tensor core reads the tile.
//
// Every mbarrier wait is bounded (see mbar_wait); there is no cluster launch and no multicast.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace helix {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kATileBytes = kBM * kBK * 2;  // 16 KiB
constexpr int kConvTableEntries = 4096;     // 8-channel chunks of the K axis (K <= 32768)

struct GemmParams {
  __half* C;
  float* partial;
  int64_t ldc;
  int64_t stride_c;
  int PM, PN, K;  // extents on the 128-row axis, on the BN axis, and the reduction
  int batch;
  int tiles_m, tiles_n, split_k, kb_per_split, num_kb;
  int total_tiles;
  int raster;
  int stages;
  int load_group;  // K slabs the TMA producer requests back to back (DRAM page locality)
  int* status;
  // convolution only
  const __half* x;
  ConvGeom g;
};

struct TileCoord {
  int m_blk, n_blk, b, ks;
};

__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int t) {
  TileCoord c;
  c.ks = t % p.split_k;
  t /= p.split_k;
  const int per_batch = p.tiles_m * p.tiles_n;
  c.b = t / per_batch;
  int r = t - c.b * per_batch;
  const int group = p.raster * p.tiles_n;
  const int gid = r / group;
  const int first_m = gid * p.raster;
  const int gm = min(p.raster, p.tiles_m - first_m);
  r -= gid * group;
  c.m_blk = first_m + r % gm;
  c.n_blk = r / gm;
  return c;
}

template <int BN>
struct SmemLayout {
  static constexpr int kBTileBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kATileBytes + kBTileBytes;
  // barriers: full[8], empty[8], tmem_full[2], tmem_empty[2]; then tmem pointer + abort flag
  static constexpr int kBarrierBytes = (8 + 8 + 2 + 2) * 8 + 16;
  static constexpr int kMaxStages = 8;
  static __host__ __device__ constexpr int tmem_cols() {
    return 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  }
};

template <int BN, bool CONV, bool SWAP, bool PARTIAL>
__global__ void __launch_bounds__(CONV ? 288 : 192, 1)
gemm_f16_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int kProducerWarps = CONV ? 4 : 1;
  constexpr int kMmaWarp = kProducerWarps;
  constexpr int kEpiWarp0 = kProducerWarps + 1;
  constexpr int kTmemCols = L::tmem_cols();
  constexpr uint32_t kIdesc = umma_idesc_f16(kBM, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* sA = smem;
  uint8_t* sB = smem + (size_t)stages * kATileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)stages * L::kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + 8;
  uint64_t* tmem_full = bars + 16;
  uint64_t* tmem_empty = bars + 18;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  uint32_t* conv_tab = reinterpret_cast<uint32_t*>(bars + 22);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], CONV ? 129 : 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    if (!CONV) tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (CONV) {
    // (r, s, c) of every 8-channel chunk of the K axis, K ordered (r, s, c)
    const int chunks = p.K >> 3;
    for (int kc = threadIdx.x; kc < chunks; kc += blockDim.x) {
      const int k = kc << 3;
      const int tap = k / p.g.C;
      const int c = k - tap * p.g.C;
      const int r = tap / p.g.S;
      const int s = tap - r * p.g.S;
      conv_tab[kc] = (uint32_t)r << 24 | (uint32_t)s << 16 | (uint32_t)c;
    }
  }
  if (warp == kMmaWarp) tmem_alloc<kTmemCols>(tmem_ptr_smem);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp < kProducerWarps) {
    // ------------------------------------------------------------------ producers
    if (!CONV) {
      if (lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
          const TileCoord tc = decode_tile(p, t);
          const int kb0 = tc.ks * p.kb_per_split;
          const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
          for (int kb = kb0; kb < kb1 && ok; kb += p.load_group) {
            // Wait for a whole group of free stages first, then request the group's slabs back to
            // back: every row then has load_group * 128 contiguous bytes in flight at once.
            const int gcount = min(p.load_group, kb1 - kb);
            int s2 = stage;
            uint32_t ph2 = phase;
            for (int g = 0; g < gcount && ok; ++g) {
              ok = mbar_wait(&empty_bar[s2], ph2 ^ 1, abort_flag, p.status);
              if (++s2 == stages) { s2 = 0; ph2 ^= 1; }
            }
            if (!ok) break;
            for (int g = 0; g < gcount; ++g) {
              mbar_arrive_expect_tx(&full_bar[stage], L::kStageBytes);
              tma_load_3d(sA + (size_t)stage * kATileBytes, &tmap_a, &full_bar[stage], (kb + g) * kBK,
                          tc.m_blk * kBM, tc.b);
              tma_load_3d(sB + (size_t)stage * L::kBTileBytes, &tmap_b, &full_bar[stage], (kb + g) * kBK,
                          tc.n_blk * BN, tc.b);
              if (++stage == stages) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
    } else {
      // Lane mapping: 8 consecutive lanes fetch the 8 16-byte chunks of one pixel's 128-byte K
      // slab, so one warp instruction touches 4 pixel rows = 4 cache lines (coalesced), and
      // writes 4 full 128-byte rows of the swizzled tile (bank-conflict free).  Warp w owns
      // rows [32w, 32w+32) of the tile in 8 passes; a thread keeps one chunk column (j) and
      // the window origin of its 8 pixels in registers.
      const int pw = threadIdx.x >> 5;       // producer warp 0..3
      const int j = lane & 7;                // 16-byte chunk of the 128-byte slab
      const int sub = lane >> 3;             // row within a pass, 0..3
      const int HoWo = p.g.Ho * p.g.Wo;
      const int chunks = p.K >> 3;
      constexpr int kInvalid = -(1 << 20);   // window origin that fails every bounds check
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x) {
        const TileCoord tc = decode_tile(p, t);
        int hi0[8], wi0[8];
        int64_t img_off[8];
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int m = tc.m_blk * kBM + pw * 32 + it * 4 + sub;
          if (m < p.PM) {
            const int n_img = m / HoWo;
            const int rem = m - n_img * HoWo;
            const int ho = rem / p.g.Wo;
            const int wo = rem - ho * p.g.Wo;
            hi0[it] = ho * p.g.stride - p.g.pad;
            wi0[it] = wo * p.g.stride - p.g.pad;
            img_off[it] = (int64_t)n_img * p.g.H * p.g.W * p.g.C;
          } else {
            hi0[it] = kInvalid;
            wi0[it] = kInvalid;
            img_off[it] = 0;
          }
        }
        const int kb0 = tc.ks * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          if (threadIdx.x == 0) {
            mbar_arrive_expect_tx(&full_bar[stage], L::kBTileBytes);
            tma_load_3d(sB + (size_t)stage * L::kBTileBytes, &tmap_b, &full_bar[stage], kb * kBK, tc.n_blk * BN, 0);
          }
          const int kc = kb * 8 + j;
          const bool k_ok = kc < chunks;
          const uint32_t e = k_ok ? conv_tab[kc] : 0u;
          const int dr = (int)(e >> 24), ds = (int)((e >> 16) & 0xFF), c0 = (int)(e & 0xFFFF);
          const uint32_t tile_base = smem_u32(sA + (size_t)stage * kATileBytes);
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int row = pw * 32 + it * 4 + sub;
            const int hi = hi0[it] + dr;
            const int wi = wi0[it] + ds;
            const bool valid = k_ok && hi >= 0 && hi < p.g.H && wi >= 0 && wi < p.g.W;
            const __half* src = valid ? p.x + img_off[it] + ((int64_t)hi * p.g.W + wi) * p.g.C + c0 : p.x;
            cp_async_16_zfill(tile_base + row * 128 + ((j ^ (row & 7)) << 4), src, valid);
          }
          // The barrier receives this thread's arrival when the copies above have landed; the
          // thread itself never blocks on them, so all stages of the ring stay in flight.
          cp_async_mbar_arrive_noinc(&full_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
      cp_async_wait<0>();  // nothing of this thread's is in flight when the CTA tears down
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++local) {
        const TileCoord tc = decode_tile(p, t);
        const int kb0 = tc.ks * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, abort_flag, p.status);
          if (!ok) break;
          // The gathered A tile was written through the generic proxy (cp.async); order those
          // writes, now visible through the barrier, before the tensor core's async-proxy reads.
          if (CONV) fence_proxy_async_smem();
          tc_fence_after_sync();
          const uint64_t da = umma_desc_sw128(smem_u32(sA + (size_t)stage * kATileBytes));
          const uint64_t db = umma_desc_sw128(smem_u32(sB + (size_t)stage * L::kBTileBytes));
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advancing 16 halves = 32 bytes along K inside the swizzle atom: +2 in the address field
            umma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, kIdesc, (kb > kb0) || (k > 0));
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter + 32)
    int local = 0;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        ((p.stride_c & 7) == 0);
    for (int t = blockIdx.x; t < p.total_tiles && ok; t += gridDim.x, ++local) {
      const TileCoord tc = decode_tile(p, t);
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tc.m_blk * kBM + quarter * 32 + lane;  // index on the 128-row (A side) axis
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      constexpr int kChunk = BN >= 32 ? 32 : 16;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += kChunk) {
        uint32_t r[kChunk];
        if constexpr (kChunk == 32) tmem_ld_32x32b_x32(taddr + c0, r);
        else tmem_ld_32x32b_x16(taddr + c0, r);
        tmem_ld_wait();
        const int col0 = tc.n_blk * BN + c0;  // index on the BN (B side) axis
        if (col0 >= p.PN) break;              // warp-uniform: nothing but padding from here on
        if constexpr (PARTIAL) {
          if (row < p.PM) {
            float* dst = p.partial + (((int64_t)tc.ks * p.batch + tc.b) * p.PM + row) * p.PN + col0;
            if (col0 + kChunk <= p.PN && (p.PN & 3) == 0) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 4)
                *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                                  __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (col0 + j < p.PN) dst[j] = __uint_as_float(r[j]);
            }
          }
        } else if constexpr (SWAP) {
          // rows index N of C, columns index M: C[m, n] with m = col, n = row
          if (row < p.PM) {
            __half* dst = p.C + (int64_t)tc.b * p.stride_c + row;
#pragma unroll
            for (int j = 0; j < kChunk; ++j)
              if (col0 + j < p.PN) dst[(int64_t)(col0 + j) * p.ldc] = __float2half_rn(__uint_as_float(r[j]));
          }
        } else {
          if (row < p.PM) {
            __half* dst = p.C + (int64_t)tc.b * p.stride_c + (int64_t)row * p.ldc + col0;
            if (vec_ok && col0 + kChunk <= p.PN) {
#pragma unroll
              for (int j = 0; j < kChunk; j += 8) {
                uint4 v;
                __half2 h0 = __floats2half2_rn(__uint_as_float(r[j + 0]), __uint_as_float(r[j + 1]));
                __half2 h1 = __floats2half2_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                __half2 h2 = __floats2half2_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                __half2 h3 = __floats2half2_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                v.x = *reinterpret_cast<uint32_t*>(&h0);
                v.y = *reinterpret_cast<uint32_t*>(&h1);
                v.z = *reinterpret_cast<uint32_t*>(&h2);
                v.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(dst + j) = v;
              }
            } else {
#pragma unroll
              for (int j = 0; j < kChunk; ++j)
                if (col0 + j < p.PN) dst[j] = __float2half_rn(__uint_as_float(r[j]));
            }
          }
        }
        __syncwarp();
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc<kTmemCols>(tmem_base);
  }
}

// Sums split-K partials in slice order (deterministic), rounds once, applies swap_ab.
__global__ void gemm_splitk_reduce_kernel(const float* __restrict__ partial, __half* __restrict__ C, int64_t ldc,
                                          int64_t stride_c, int PM, int PN, int batch, int split_k, int swap) {
  const int64_t per = (int64_t)PM * PN;
  const int64_t total = per * batch;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float s = 0.0f;
    for (int ks = 0; ks < split_k; ++ks) s += partial[(int64_t)ks * total + i];
    const int b = (int)(i / per);
    const int64_t rem = i - (int64_t)b * per;
    const int row = (int)(rem / PN), col = (int)(rem - (int64_t)row * PN);
    const int64_t o = swap ? (int64_t)col * ldc + row : (int64_t)row * ldc + col;
    C[(int64_t)b * stride_c + o] = __float2half_rn(s);
  }
}

// ===================================================================== host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
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

// K-major fp16 matrix [batch][rows][K] with leading dimension ld and batch stride bs (elements);
// box = 64 halves x box_rows x 1, 128-byte swizzle, out-of-bounds elements read as zero.
static int make_tmap(CUtensorMap* map, const void* base, int64_t K, int64_t rows, int64_t batch, int64_t ld, int64_t bs,
                     int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return HELIX_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 7) || (batch > 1 && (bs & 7))) return HELIX_ERR_ALIGN;
  if (batch <= 1) bs = rows * ld;
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(batch, 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HELIX_OK : HELIX_ERR_CUDA;
}

static const int kTileNs[] = {256, 128, 64, 32, 16};
constexpr int kNumTileNs = sizeof(kTileNs) / sizeof(kTileNs[0]);

int gemm_f16_num_configs() { return kNumTileNs * 2; }
void gemm_f16_get_config(int idx, helix_cfg_t* out) {
  out->op = HELIX_OP_GEMM_F16;
  out->tile_m = kBM;
  out->tile_n = kTileNs[idx % kNumTileNs];
  out->tile_k = kBK;
  out->stages = 0;
  out->cta_group = 1;
  out->split_k = 1;
  out->swap_ab = idx / kNumTileNs;
  out->raster = 8;
}

static int max_stages(int bn, bool conv) {
  const int budget = 227 * 1024 - 1024 /*alignment slack*/ - 256 /*barriers*/ - (conv ? kConvTableEntries * 4 : 0);
  int s = budget / (kATileBytes + bn * kBK * 2);
  return std::min(s, 8);
}

// Cycle estimate of one K slab: the slower of tensor issue (BN/2 cycles per K=16 step) and the
// shared-memory read of both operand tiles at 128 bytes per cycle.
static double slab_cycles(int bn) {
  const double mma = 4.0 * bn / 2.0;
  const double smem = (kATileBytes + bn * kBK * 2) / 128.0;
  return std::max(mma, smem);
}

void gemm_f16_default_config(int M, int N, int K, int batch, int sm_count, bool conv, helix_cfg_t* out) {
  *out = helix_cfg_t{};
  out->op = conv ? HELIX_OP_CONV_F16 : HELIX_OP_GEMM_F16;
  out->tile_m = kBM;
  out->tile_k = kBK;
  out->cta_group = 1;
  out->raster = 8;
  const int num_kb = (K + kBK - 1) / kBK;
  double best = 1e30;
  const double hbm_bytes_per_cycle = 3400.0;  // ~6.5 TB/s at ~1.9 GHz
  for (int swap = 0; swap <= (conv ? 0 : 1); ++swap) {
    const int pm = swap ? N : M, pn = swap ? M : N;
    for (int i = 0; i < kNumTileNs; ++i) {
      const int bn = kTileNs[i];
      if (bn > 16 && bn / 2 >= pn && i + 1 < kNumTileNs) continue;  // a smaller tile covers PN as well
      const int64_t tiles = (int64_t)((pm + kBM - 1) / kBM) * ((pn + bn - 1) / bn) * batch;
      for (int sk = 1; sk <= 16; sk *= 2) {
        if (sk > 1 && (num_kb / sk < 4)) break;
        const int kbs = (num_kb + sk - 1) / sk;
        const int64_t waves = (tiles * sk + sm_count - 1) / sm_count;
        // one SM streams operands at a bounded rate, so few fat CTAs cannot saturate HBM
        const double tile_bytes = (double)kbs * 128.0 * (std::min(pm, kBM) + std::min(pn, bn));
        const double per_tile = std::max(kbs * slab_cycles(bn), tile_bytes / 56.0) + 700.0;
        double cyc = waves * per_tile;
        const double bytes = 2.0 * batch * ((double)M * K + (double)N * K + (double)M * N) +
                             (sk > 1 ? 4.0 * sk * batch * (double)M * N : 0.0);
        cyc = std::max(cyc, bytes / hbm_bytes_per_cycle);
        // the reduction kernel runs after the GEMM: reads sk fp32 partials, writes fp16
        if (sk > 1) cyc += 3000.0 + batch * (double)M * N * (4.0 * sk + 2.0) / hbm_bytes_per_cycle;
        if (cyc < best) {
          best = cyc;
          out->tile_n = bn;
          out->split_k = sk;
          out->swap_ab = swap;
        }
      }
    }
  }
  out->stages = max_stages(out->tile_n, conv);
}

size_t gemm_f16_workspace_bytes(const helix_cfg_t* cfg, int M, int N, int K, int batch) {
  if (!cfg || cfg->split_k <= 1) return 0;
  return (size_t)cfg->split_k * std::max(batch, 1) * (size_t)M * N * sizeof(float);
}

template <int BN, bool CONV>
static cudaError_t launch_variant(bool swap, bool partial, const CUtensorMap& ta, const CUtensorMap& tb,
                                  const GemmParams& p, int grid, size_t smem, cudaStream_t stream) {
  constexpr int threads = CONV ? 288 : 192;
#define HELIX_LAUNCH(SW, PA)                                                                             \
  do {                                                                                                   \
    auto kern = gemm_f16_tc_kernel<BN, CONV, SW, PA>;                                                    \
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    if (e != cudaSuccess) return e;                                                                      \
    kern<<<grid, threads, smem, stream>>>(ta, tb, p);                                                    \
    return cudaGetLastError();                                                                           \
  } while (0)
  if (partial) HELIX_LAUNCH(false, true);
  if constexpr (!CONV) {
    if (swap) HELIX_LAUNCH(true, false);
  }
  HELIX_LAUNCH(false, false);
#undef HELIX_LAUNCH
}

static int launch_common(const helix_cfg_t& cfg, bool conv, const CUtensorMap& ta, const CUtensorMap& tb,
                         GemmParams& p, void* C, int64_t ldc, int64_t sc, void* ws, size_t ws_bytes, int sm_count,
                         cudaStream_t stream, int64_t* launches) {
  const int bn = cfg.tile_n;
  p.tiles_m = (p.PM + kBM - 1) / kBM;
  p.tiles_n = (p.PN + bn - 1) / bn;
  p.num_kb = (p.K + kBK - 1) / kBK;
  p.split_k = std::max(1, std::min(cfg.split_k, p.num_kb));
  p.kb_per_split = (p.num_kb + p.split_k - 1) / p.split_k;
  p.split_k = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;  // no empty slices
  const int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.batch * p.split_k;
  if (total <= 0 || total > 0x7fffffff) return HELIX_ERR_INVALID;
  p.total_tiles = (int)total;
  p.raster = cfg.raster > 0 ? cfg.raster : 8;
  const int smax = max_stages(bn, conv);
  p.stages = cfg.stages > 0 ? std::min(cfg.stages, smax) : smax;
  if (p.stages < (conv ? 3 : 2)) return HELIX_ERR_UNSUPPORTED;
  p.load_group = std::max(1, std::min(cfg.load_group > 0 ? cfg.load_group : 1, p.stages / 2));
  const bool partial = p.split_k > 1;
  if (partial) {
    const size_t need = (size_t)p.split_k * p.batch * (size_t)p.PM * p.PN * sizeof(float);
    if (!ws || ws_bytes < need) return HELIX_ERR_WORKSPACE;
    p.partial = static_cast<float*>(ws);
  }
  p.C = static_cast<__half*>(C);
  p.ldc = ldc;
  p.stride_c = sc;
  const int grid = (int)std::min<int64_t>(total, sm_count);
  const size_t smem = 1024 + (size_t)p.stages * (kATileBytes + bn * kBK * 2) + 256 + (conv ? kConvTableEntries * 4 : 0);
  cudaError_t e = cudaErrorInvalidValue;
  const bool swap = cfg.swap_ab != 0;
#define HELIX_BN_CASE(BNV)                                                                                     \
  case BNV:                                                                                                    \
    e = conv ? launch_variant<BNV, true>(false, partial, ta, tb, p, grid, smem, stream)                        \
             : launch_variant<BNV, false>(swap, partial, ta, tb, p, grid, smem, stream);                       \
    break;
  switch (bn) {
    HELIX_BN_CASE(256)
    HELIX_BN_CASE(128)
    HELIX_BN_CASE(64)
    HELIX_BN_CASE(32)
    HELIX_BN_CASE(16)
    default:
      return HELIX_ERR_UNSUPPORTED;
  }
#undef HELIX_BN_CASE
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  if (partial) {
    const int64_t n = (int64_t)p.PM * p.PN * p.batch;
    const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)sm_count * 8);
    gemm_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.partial, p.C, ldc, sc, p.PM, p.PN, p.batch, p.split_k,
                                                         swap ? 1 : 0);
    if (cudaGetLastError() != cudaSuccess) return HELIX_ERR_CUDA;
    ++*launches;
  }
  return HELIX_OK;
}

int gemm_f16_launch(const helix_cfg_t* cfg_in, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                    int64_t ldc, int M, int N, int K, int batch, int64_t sa, int64_t sb, int64_t sc, void* ws,
                    size_t ws_bytes, int* status_dev, int sm_count, cudaStream_t stream, int64_t* launches) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return HELIX_ERR_INVALID;
  if (batch <= 0) batch = 1;
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = K;
  if (ldc == 0) ldc = N;
  if (sa == 0) sa = (int64_t)M * lda;
  if (sb == 0) sb = (int64_t)N * ldb;
  if (sc == 0) sc = (int64_t)M * ldc;
  helix_cfg_t cfg;
  if (cfg_in && cfg_in->tile_m != 0) {
    cfg = *cfg_in;
  } else {
    gemm_f16_default_config(M, N, K, batch, sm_count, false, &cfg);
    if (cfg.split_k > 1 && (!ws || ws_bytes < gemm_f16_workspace_bytes(&cfg, M, N, K, batch))) cfg.split_k = 1;
  }
  if (cfg.tile_m != kBM || cfg.cta_group > 1) return HELIX_ERR_UNSUPPORTED;
  const bool swap = cfg.swap_ab != 0;
  GemmParams p{};
  p.PM = swap ? N : M;
  p.PN = swap ? M : N;
  p.K = K;
  p.batch = batch;
  p.status = status_dev;
  CUtensorMap ta, tb;
  int rc;
  if (!swap) {
    if ((rc = make_tmap(&ta, A, K, M, batch, lda, sa, kBM)) != HELIX_OK) return rc;
    if ((rc = make_tmap(&tb, B, K, N, batch, ldb, sb, cfg.tile_n)) != HELIX_OK) return rc;
  } else {
    if ((rc = make_tmap(&ta, B, K, N, batch, ldb, sb, kBM)) != HELIX_OK) return rc;
    if ((rc = make_tmap(&tb, A, K, M, batch, lda, sa, cfg.tile_n)) != HELIX_OK) return rc;
  }
  return launch_common(cfg, false, ta, tb, p, C, ldc, sc, ws, ws_bytes, sm_count, stream, launches);
}

int conv_f16_launch(const helix_cfg_t* cfg_in, const void* x, const void* w, void* y, const ConvGeom& g, void* ws,
                    size_t ws_bytes, int* status_dev, int sm_count, cudaStream_t stream, int64_t* launches) {
  if (!x || !w || !y || g.NB <= 0 || g.H <= 0 || g.W <= 0 || g.C <= 0 || g.KO <= 0 || g.R <= 0 || g.S <= 0 ||
      g.stride <= 0 || g.pad < 0 || g.Ho <= 0 || g.Wo <= 0)
    return HELIX_ERR_INVALID;
  if ((g.C & 7) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return HELIX_ERR_ALIGN;
  const int64_t M64 = (int64_t)g.NB * g.Ho * g.Wo;
  const int64_t K64 = (int64_t)g.R * g.S * g.C;
  if (M64 > 0x7fffffff || K64 > (int64_t)kConvTableEntries * 8 || g.R > 255 || g.S > 255 || g.C > 65535)
    return HELIX_ERR_UNSUPPORTED;
  const int M = (int)M64, K = (int)K64, N = g.KO;
  // A 1x1, stride-1, unpadded convolution is exactly a GEMM over the pixel list.
  if (g.R == 1 && g.S == 1 && g.stride == 1 && g.pad == 0)
    return gemm_f16_launch(cfg_in && cfg_in->tile_m ? cfg_in : nullptr, x, g.C, w, g.C, y, N, M, N, K, 1, 0, 0, 0, ws,
                           ws_bytes, status_dev, sm_count, stream, launches);
  helix_cfg_t cfg;
  if (cfg_in && cfg_in->tile_m != 0) {
    cfg = *cfg_in;
  } else {
    gemm_f16_default_config(M, N, K, 1, sm_count, true, &cfg);
    if (cfg.split_k > 1 && (!ws || ws_bytes < gemm_f16_workspace_bytes(&cfg, M, N, K, 1))) cfg.split_k = 1;
  }
  if (cfg.tile_m != kBM || cfg.cta_group > 1 || cfg.swap_ab) return HELIX_ERR_UNSUPPORTED;
  GemmParams p{};
  p.PM = M;
  p.PN = N;
  p.K = K;
  p.batch = 1;
  p.status = status_dev;
  p.x = static_cast<const __half*>(x);
  p.g = g;
  CUtensorMap tb;
  int rc;
  if ((rc = make_tmap(&tb, w, K, N, 1, K, 0, cfg.tile_n)) != HELIX_OK) return rc;
  return launch_common(cfg, true, tb, tb, p, y, N, 0, ws, ws_bytes, sm_count, stream, launches);
}

}  // namespace helix
