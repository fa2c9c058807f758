// True-fp32 SIMT GEMM: C[M,N] = A * B with FFMA only (no TF32, no tensor cores).
//
// Counterpart of the reference's mySgemmCPAsyncTemplate (src_template/Ampere_FP32/sgemm.cu
// :97-350).  B is K x N row-major; A is M x K row-major (the x86 template's layout,
// scripts/x86_CPU/profile_x86_CPU.py:27-29) or K x M when trans_a is set (what the reference
// kernel is handed, sgemm.cu:138).  Every output element accumulates k = 0, 1, 2, ... in one
// fp32 register with one fused multiply-add per step, so the result is bit-identical to an
// fmaf() chain on the host.
//
// CTA tile BM x BN x BK, (BM/TM)*(BN/TN) threads, each thread a TM x TN register block split
// into 4-wide quads that are strided across the tile (conflict-free float4 reads from shared
// memory).  A is staged K-major ([BK][BM]) so both operands are read as float4 along the
// output dimension.  Global loads of slab k+1 are issued into registers before the FFMA loop
// of slab k and written to the other shared buffer afterwards (one __syncthreads per slab).
#include "common.cuh"
#include "kernels.h"

namespace helix {

template <int BM, int BN, int BK, int TM, int TN>
struct SgemmTraits {
  static constexpr int kThreadsM = BM / TM;
  static constexpr int kThreadsN = BN / TN;
  static constexpr int kThreads = kThreadsM * kThreadsN;
  static constexpr int kAElems = BM * BK / kThreads;  // floats of A per thread per slab
  static constexpr int kBElems = BN * BK / kThreads;
  static_assert(TM % 4 == 0 && TN % 4 == 0, "register block is made of 4-wide quads");
  static_assert(kAElems % 4 == 0 && kBElems % 4 == 0, "whole float4s per thread");
};

template <int BM, int BN, int BK, int TM, int TN, bool TRANS_A, bool VEC>
__global__ void __launch_bounds__(SgemmTraits<BM, BN, BK, TM, TN>::kThreads)
sgemm_f32_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ B, int64_t ldb,
                 float* __restrict__ C, int64_t ldc, int M, int N, int K) {
  using T = SgemmTraits<BM, BN, BK, TM, TN>;
  constexpr int NT = T::kThreads;
  constexpr int A4 = T::kAElems / 4;
  constexpr int B4 = T::kBElems / 4;
  __shared__ __align__(16) float sA[2][BK][BM + 4];
  __shared__ __align__(16) float sB[2][BK][BN + 4];

  const int tid = threadIdx.x;
  const int tn = tid % T::kThreadsN;
  const int tm = tid / T::kThreadsN;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  float4 ra[A4], rb[B4];
  auto a_swz = [](int kk) { return ((kk >> 2) & 3) << 2; };   // column XOR of sA row kk (multiple of 4)

  // ---- global -> registers for slab starting at k0 (zero fill outside the matrix)
  auto load_global = [&](int k0) {
#pragma unroll
    for (int v = 0; v < A4; ++v) {
      const int f = (v * NT + tid);  // float4 index inside the slab
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (TRANS_A) {
        // A is K x M: a float4 runs along M
        const int kk = f / (BM / 4), mm = (f % (BM / 4)) * 4;
        const int gk = k0 + kk, gm = m0 + mm;
        if (gk < K) {
          const float* p = A + (int64_t)gk * lda + gm;
          if (VEC && gm + 3 < M) val = *reinterpret_cast<const float4*>(p);
          else {
            if (gm + 0 < M) val.x = p[0];
            if (gm + 1 < M) val.y = p[1];
            if (gm + 2 < M) val.z = p[2];
            if (gm + 3 < M) val.w = p[3];
          }
        }
      } else {
        // A is M x K: a float4 runs along K
        const int mm = f / (BK / 4), kk = (f % (BK / 4)) * 4;
        const int gk = k0 + kk, gm = m0 + mm;
        if (gm < M) {
          const float* p = A + (int64_t)gm * lda + gk;
          if (VEC && gk + 3 < K) val = *reinterpret_cast<const float4*>(p);
          else {
            if (gk + 0 < K) val.x = p[0];
            if (gk + 1 < K) val.y = p[1];
            if (gk + 2 < K) val.z = p[2];
            if (gk + 3 < K) val.w = p[3];
          }
        }
      }
      ra[v] = val;
    }
#pragma unroll
    for (int v = 0; v < B4; ++v) {
      const int f = (v * NT + tid);
      const int kk = f / (BN / 4), nn = (f % (BN / 4)) * 4;
      const int gk = k0 + kk, gn = n0 + nn;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gk < K) {
        const float* p = B + (int64_t)gk * ldb + gn;
        if (VEC && gn + 3 < N) val = *reinterpret_cast<const float4*>(p);
        else {
          if (gn + 0 < N) val.x = p[0];
          if (gn + 1 < N) val.y = p[1];
          if (gn + 2 < N) val.z = p[2];
          if (gn + 3 < N) val.w = p[3];
        }
      }
      rb[v] = val;
    }
  };
  // ---- registers -> shared buffer `buf`
  auto store_shared = [&](int buf) {
#pragma unroll
    for (int v = 0; v < A4; ++v) {
      const int f = (v * NT + tid);
      if (TRANS_A) {
        const int kk = f / (BM / 4), mm = (f % (BM / 4)) * 4;
        *reinterpret_cast<float4*>(&sA[buf][kk][mm ^ a_swz(kk)]) = ra[v];
      } else {
        // the four k values of a float4 go to four rows; rows kk, kk+4, kk+8, kk+12 of one warp's
        // stores would share banks pairwise, so the column is XOR-ed with a multiple of 4 that
        // depends on kk / 4 (whole float4 groups move, the later float4 reads stay aligned)
        const int mm = f / (BK / 4), kk = (f % (BK / 4)) * 4;
        const int col = mm ^ a_swz(kk);
        sA[buf][kk + 0][col] = ra[v].x;
        sA[buf][kk + 1][col] = ra[v].y;
        sA[buf][kk + 2][col] = ra[v].z;
        sA[buf][kk + 3][col] = ra[v].w;
      }
    }
#pragma unroll
    for (int v = 0; v < B4; ++v) {
      const int f = (v * NT + tid);
      const int kk = f / (BN / 4), nn = (f % (BN / 4)) * 4;
      *reinterpret_cast<float4*>(&sB[buf][kk][nn]) = rb[v];
    }
  };

  const int num_slabs = (K + BK - 1) / BK;
  if (num_slabs > 0) {
    load_global(0);
    store_shared(0);
  }
  __syncthreads();

  for (int s = 0; s < num_slabs; ++s) {
    const int buf = s & 1;
    if (s + 1 < num_slabs) load_global((s + 1) * BK);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], bv[TN];
#pragma unroll
      for (int q = 0; q < TM / 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(&sA[buf][kk][((q * T::kThreadsM + tm) * 4) ^ a_swz(kk)]);
        av[q * 4 + 0] = t.x; av[q * 4 + 1] = t.y; av[q * 4 + 2] = t.z; av[q * 4 + 3] = t.w;
      }
#pragma unroll
      for (int q = 0; q < TN / 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(&sB[buf][kk][(q * T::kThreadsN + tn) * 4]);
        bv[q * 4 + 0] = t.x; bv[q * 4 + 1] = t.y; bv[q * 4 + 2] = t.z; bv[q * 4 + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    if (s + 1 < num_slabs) store_shared(buf ^ 1);
    __syncthreads();
  }

  // ---- epilogue: quads are strided across the tile
#pragma unroll
  for (int qi = 0; qi < TM / 4; ++qi)
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int gm = m0 + (qi * T::kThreadsM + tm) * 4 + ii;
      if (gm >= M) continue;
#pragma unroll
      for (int qj = 0; qj < TN / 4; ++qj) {
        const int gn = n0 + (qj * T::kThreadsN + tn) * 4;
        float* p = C + (int64_t)gm * ldc + gn;
        const float* a = &acc[qi * 4 + ii][qj * 4];
        if (VEC && gn + 3 < N) *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
        else {
          if (gn + 0 < N) p[0] = a[0];
          if (gn + 1 < N) p[1] = a[1];
          if (gn + 2 < N) p[2] = a[2];
          if (gn + 3 < N) p[3] = a[3];
        }
      }
    }
}

struct SgemmCfg { int bm, bn, bk, tm, tn; };
static const SgemmCfg kSgemmCfgs[] = {
    {128, 128, 16, 8, 8}, {128, 64, 16, 8, 4}, {64, 128, 16, 4, 8}, {64, 64, 16, 4, 4}, {32, 64, 16, 4, 4},
};
constexpr int kNumSgemmCfgs = sizeof(kSgemmCfgs) / sizeof(kSgemmCfgs[0]);

int sgemm_f32_num_configs() { return kNumSgemmCfgs; }
void sgemm_f32_get_config(int idx, helix_cfg_t* out) {
  *out = helix_cfg_t{};
  out->op = HELIX_OP_GEMM_F32;
  out->tile_m = kSgemmCfgs[idx].bm;
  out->tile_n = kSgemmCfgs[idx].bn;
  out->tile_k = kSgemmCfgs[idx].bk;
  out->thread_m = kSgemmCfgs[idx].tm;
  out->thread_n = kSgemmCfgs[idx].tn;
  out->stages = 2;
  out->cta_group = 1;
  out->split_k = 1;
}

// Largest tile that still yields about two CTAs per SM, else the smallest tile.
void sgemm_f32_default_config(int M, int N, int sm_count, helix_cfg_t* out) {
  int pick = kNumSgemmCfgs - 1;
  for (int i = 0; i < kNumSgemmCfgs; ++i) {
    const int64_t tiles = (int64_t)((M + kSgemmCfgs[i].bm - 1) / kSgemmCfgs[i].bm) *
                          ((N + kSgemmCfgs[i].bn - 1) / kSgemmCfgs[i].bn);
    if (tiles >= 2 * (int64_t)sm_count) { pick = i; break; }
  }
  sgemm_f32_get_config(pick, out);
}

template <int BM, int BN, int BK, int TM, int TN>
static void launch_sgemm(const float* A, int64_t lda, bool trans_a, const float* B, int64_t ldb, float* C,
                         int64_t ldc, int M, int N, int K, bool vec, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  constexpr int NT = SgemmTraits<BM, BN, BK, TM, TN>::kThreads;
  if (trans_a) {
    if (vec) sgemm_f32_kernel<BM, BN, BK, TM, TN, true, true><<<grid, NT, 0, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
    else sgemm_f32_kernel<BM, BN, BK, TM, TN, true, false><<<grid, NT, 0, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
  } else {
    if (vec) sgemm_f32_kernel<BM, BN, BK, TM, TN, false, true><<<grid, NT, 0, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
    else sgemm_f32_kernel<BM, BN, BK, TM, TN, false, false><<<grid, NT, 0, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
  }
}

int sgemm_f32_launch(const helix_cfg_t* cfg, const float* A, int64_t lda, int trans_a, const float* B, int64_t ldb,
                     float* C, int64_t ldc, int M, int N, int K, int sm_count, cudaStream_t stream,
                     int64_t* launches) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K < 0) return HELIX_ERR_INVALID;
  if (lda == 0) lda = trans_a ? M : K;
  if (ldb == 0) ldb = N;
  if (ldc == 0) ldc = N;
  const bool vec = ((lda & 3) == 0) && ((ldb & 3) == 0) && ((ldc & 3) == 0) &&
                   ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((reinterpret_cast<uintptr_t>(B) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
  int bm, bn;
  if (cfg && cfg->tile_m != 0) {
    bm = cfg->tile_m;
    bn = cfg->tile_n;
  } else {
    helix_cfg_t def{};
    sgemm_f32_default_config(M, N, sm_count, &def);
    bm = def.tile_m;
    bn = def.tile_n;
  }
  const bool ta = trans_a != 0;
  if (bm == 128 && bn == 128) launch_sgemm<128, 128, 16, 8, 8>(A, lda, ta, B, ldb, C, ldc, M, N, K, vec, stream);
  else if (bm == 128 && bn == 64) launch_sgemm<128, 64, 16, 8, 4>(A, lda, ta, B, ldb, C, ldc, M, N, K, vec, stream);
  else if (bm == 64 && bn == 128) launch_sgemm<64, 128, 16, 4, 8>(A, lda, ta, B, ldb, C, ldc, M, N, K, vec, stream);
  else if (bm == 64 && bn == 64) launch_sgemm<64, 64, 16, 4, 4>(A, lda, ta, B, ldb, C, ldc, M, N, K, vec, stream);
  else if (bm == 32 && bn == 64) launch_sgemm<32, 64, 16, 4, 4>(A, lda, ta, B, ldb, C, ldc, M, N, K, vec, stream);
  else return HELIX_ERR_UNSUPPORTED;
  ++*launches;
  return cudaGetLastError() == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
}

}  // namespace helix
