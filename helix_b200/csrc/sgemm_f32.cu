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
  static_assert(kThreadsM % 4 == 0 && kThreadsN % 8 == 0, "a warp covers 4 x 8 threads of the grid");
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

  // a warp covers 4 x 8 threads of the kThreadsM x kThreadsN grid, a half-warp 4 x 4: a 128-bit shared
  // load is served half-warp by half-warp, and 4 distinct float4 per half cost one pass instead of two
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int kWarpsN = T::kThreadsN / 8;
  const int tn = (warp % kWarpsN) * 8 + (lane & 3) + 4 * (lane >> 4);
  const int tm = (warp / kWarpsN) * 4 + ((lane >> 2) & 3);
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

// ---------------------------------------------------------------------------------------------
// Pipelined variant for 16-byte-aligned operands: cp.async straight from global to shared memory
// through a ring of STAGES slabs (no register staging, one __syncthreads per slab, loads issued
// STAGES-1 slabs ahead).  Both operands are staged K-major as above.  B and a K x M A (trans_a)
// arrive as 16-byte copies.  A row-major M x K A with register blocks of up to 32 accumulators arrives
// as 8-byte copies of two consecutive k and is staged as k pairs ([BK/2][BM + 2][2]): the eight floats
// a thread needs for a quad of rows and one k pair are contiguous, so it reads them with two 16-byte
// loads per pair -- the same number of shared loads per FFMA as the K-major layout, without a
// transposing copy per element (1024^3, 128 x 64 tile: 66.1 -> 60.1 us).  With 8 x 8 blocks the pair
// fragments cost 16 more registers and the kernel gets slower (4096^3: 2615 -> 2880 us; 2797 us when the
// next pair is fetched stripe by stripe into the registers the current pair's last step frees), so there the
// copy itself transposes, one 4-byte cp.async per element into the K-major layout.
// Rows outside the matrix and the K tail are zero-filled by the copy's source size.
template <int BM, int BN, int BK, int TM, int TN, int STAGES, bool TRANS_A>
struct SgemmPipeTraits {
  static constexpr int kThreadsM = BM / TM;
  static constexpr int kThreadsN = BN / TN;
  static constexpr int kThreads = kThreadsM * kThreadsN;
  // K x M A: staged K-major, one row of BM + 4 floats per k.  M x K A: staged as k pairs, [BK/2][BM + 2][2]
  // (the two k of an 8-byte copy stay together; BM + 2 = 2 mod 16 spreads the copies of a warp over all banks)
  static constexpr bool kPair = !TRANS_A && TM * TN <= 32;   // with 64 accumulators the pair fragments cost too many registers (measured slower)
  static constexpr int kARow = BM + 4;                         // floats per shared row (one k) of A, K-major
  static constexpr int kARowP = BM + 2;                        // rows (m) per k pair, pair-major
  static constexpr int kBRow = BN + 4;
  static constexpr int kAStage = kPair ? BK * kARowP : BK * kARow;   // floats per stage
  static constexpr int kBStage = BK * kBRow;
  static constexpr int kSmemBytes = STAGES * (kAStage + kBStage) * 4;
  static constexpr int kA4 = BM * BK / 4 / kThreads;           // 16-byte copies of A per thread per slab (K x M A)
  static constexpr int kA1 = BM * BK / kThreads;               // 4-byte copies of A per thread per slab (M x K A, K-major)
  static constexpr int kA2 = BM * BK / 2 / kThreads;           // 8-byte copies of A per thread per slab (M x K A)
  static constexpr int kB4 = BN * BK / 4 / kThreads;
  static_assert(TM % 4 == 0 && TN % 4 == 0 && BK % 8 == 0, "4-wide quads, steps unrolled by eight");
  static_assert(kThreadsM % 4 == 0 && kThreadsN % 8 == 0, "a warp covers 4 x 8 threads of the grid");
  static_assert((BM * BK / 4) % kThreads == 0 && (BN * BK / 4) % kThreads == 0, "whole copies per thread");
};

__device__ __forceinline__ void cp_async_16_bytes(uint32_t smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes)
               : "memory");
}

__device__ __forceinline__ void cp_async_4_bytes(uint32_t smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes)
               : "memory");
}

__device__ __forceinline__ void cp_async_8_bytes(uint32_t smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes)
               : "memory");
}

template <int BM, int BN, int BK, int TM, int TN, int STAGES, bool TRANS_A, int MIN_CTAS>
__global__ void __launch_bounds__(SgemmPipeTraits<BM, BN, BK, TM, TN, STAGES, TRANS_A>::kThreads, MIN_CTAS)
sgemm_f32_pipe_kernel(const float* __restrict__ A, int64_t lda, const float* __restrict__ B, int64_t ldb,
                      float* __restrict__ C, int64_t ldc, int M, int N, int K) {
  using T = SgemmPipeTraits<BM, BN, BK, TM, TN, STAGES, TRANS_A>;
  constexpr int NT = T::kThreads;
  extern __shared__ __align__(16) float smem_f[];
  float* sA = smem_f;
  float* sB = smem_f + STAGES * T::kAStage;
  const uint32_t sA_u = smem_u32(sA), sB_u = smem_u32(sB);

  // Thread grid kThreadsM x kThreadsN; a warp covers 4 x 8 of it and each half-warp 4 x 4, so that a
  // 16-byte shared load touches at most 64 distinct bytes per half-warp: a 128-bit shared load is
  // served half-warp by half-warp, 128 distinct bytes per pass (measured: 16 lanes reading 16
  // different float4 cost two passes per half)
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  constexpr int kWarpsN = T::kThreadsN / 8;
  const int tn = (warp % kWarpsN) * 8 + (lane & 3) + 4 * (lane >> 4);
  const int tm = (warp / kWarpsN) * 4 + ((lane >> 2) & 3);
  auto row_of = [&](int i) { return ((i >> 2) * T::kThreadsM + tm) * 4 + (i & 3); };   // quads of rows
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  // Copies of an interior tile and a full slab need no bounds work: every thread keeps one running
  // pointer per operand (advanced once per slab) and its passes are a fixed stride apart.
  const bool interior = (m0 + BM <= M) && (n0 + BN <= N);
  constexpr int kAPassRows = TRANS_A ? NT / (BM / 4) : (T::kPair ? NT / (BK / 2) : NT / BK);   // k rows (K x M A) or m rows (M x K A) per pass
  constexpr int kBPassRows = NT / (BN / 4);
  const int a_r = TRANS_A ? tid / (BM / 4) : (T::kPair ? tid / (BK / 2) : tid / BK);               // row of the first pass
  const int a_c = TRANS_A ? (tid % (BM / 4)) * 4 : (T::kPair ? (tid % (BK / 2)) * 2 : tid % BK);   // column (m for K x M, even k for M x K)
  const int b_r = tid / (BN / 4), b_c = (tid % (BN / 4)) * 4;
  const float* a_run = TRANS_A ? A + (int64_t)a_r * lda + (m0 + a_c) : A + (int64_t)(m0 + a_r) * lda + a_c;
  const float* b_run = B + (int64_t)b_r * ldb + (n0 + b_c);
  const int64_t a_pass = (int64_t)kAPassRows * lda;
  const int64_t b_pass = (int64_t)kBPassRows * ldb;
  const int64_t a_slab = TRANS_A ? (int64_t)BK * lda : (int64_t)BK;
  const int64_t b_slab = (int64_t)BK * ldb;
  const uint32_t a_dst = sA_u + (uint32_t)(TRANS_A ? a_r * T::kARow + a_c : (T::kPair ? ((a_c >> 1) * T::kARowP + a_r) * 2 : a_c * T::kARow + a_r)) * 4u;
  const uint32_t b_dst = sB_u + (uint32_t)(b_r * T::kBRow + b_c) * 4u;
  constexpr uint32_t kADstPass = (TRANS_A ? kAPassRows * T::kARow : (T::kPair ? kAPassRows * 2 : kAPassRows)) * 4u;
  constexpr uint32_t kBDstPass = kBPassRows * T::kBRow * 4u;
  int slabs_issued = 0;      // a_run / b_run point at slab `slabs_issued`

  auto issue = [&](int slab, int stage) {
    const int k0 = slab * BK;
    if (interior && k0 + BK <= K && slab == slabs_issued) {
      const uint32_t ad = a_dst + (uint32_t)(stage * T::kAStage) * 4u;
      const uint32_t bd = b_dst + (uint32_t)(stage * T::kBStage) * 4u;
      if (TRANS_A) {
#pragma unroll
        for (int v = 0; v < T::kA4; ++v)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ad + v * kADstPass), "l"(a_run + v * a_pass) : "memory");
      } else if (T::kPair) {
#pragma unroll
        for (int v = 0; v < T::kA2; ++v)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(ad + v * kADstPass), "l"(a_run + v * a_pass) : "memory");
      } else {
#pragma unroll
        for (int v = 0; v < T::kA1; ++v)
          asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ad + v * kADstPass), "l"(a_run + v * a_pass) : "memory");
      }
#pragma unroll
      for (int v = 0; v < T::kB4; ++v)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(bd + v * kBDstPass), "l"(b_run + v * b_pass) : "memory");
      a_run += a_slab;
      b_run += b_slab;
      ++slabs_issued;
      return;
    }
    if (TRANS_A) {
#pragma unroll
      for (int v = 0; v < T::kA4; ++v) {
        const int f = v * NT + tid;
        const int kk = f / (BM / 4), mm = (f % (BM / 4)) * 4;
        const int gk = k0 + kk, gm = m0 + mm;
        const int bytes = gk < K ? max(0, min(4, M - gm)) * 4 : 0;
        const float* src = bytes ? A + (int64_t)gk * lda + gm : A;
        cp_async_16_bytes(sA_u + (uint32_t)(stage * T::kAStage + kk * T::kARow + mm) * 4u, src, bytes);
      }
    } else if (T::kPair) {
#pragma unroll
      for (int v = 0; v < T::kA2; ++v) {
        const int mm = a_r + v * kAPassRows, kk = a_c;
        const int gk = k0 + kk, gm = m0 + mm;
        const int bytes = gm < M ? max(0, min(2, K - gk)) * 4 : 0;
        const float* src = bytes ? A + (int64_t)gm * lda + gk : A;
        cp_async_8_bytes(sA_u + (uint32_t)(stage * T::kAStage + ((kk >> 1) * T::kARowP + mm) * 2) * 4u, src, bytes);
      }
    } else {
#pragma unroll
      for (int v = 0; v < T::kA1; ++v) {
        const int mm = a_r + v * kAPassRows, kk = a_c;
        const int gk = k0 + kk, gm = m0 + mm;
        const int bytes = (gm < M && gk < K) ? 4 : 0;
        const float* src = bytes ? A + (int64_t)gm * lda + gk : A;
        cp_async_4_bytes(sA_u + (uint32_t)(stage * T::kAStage + kk * T::kARow + mm) * 4u, src, bytes);
      }
    }
#pragma unroll
    for (int v = 0; v < T::kB4; ++v) {
      const int f = v * NT + tid;
      const int kk = f / (BN / 4), nn = (f % (BN / 4)) * 4;
      const int gk = k0 + kk, gn = n0 + nn;
      const int bytes = gk < K ? max(0, min(4, N - gn)) * 4 : 0;
      const float* src = bytes ? B + (int64_t)gk * ldb + gn : B;
      cp_async_16_bytes(sB_u + (uint32_t)(stage * T::kBStage + kk * T::kBRow + nn) * 4u, src, bytes);
    }
  };

  const int num_slabs = (K + BK - 1) / BK;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_slabs) issue(s, s);
    cp_async_commit();
  }

  int stage = 0;
  for (int s = 0; s < num_slabs; ++s) {
    cp_async_wait<STAGES - 2>();      // slab s has landed (this thread's copies) ...
    __syncthreads();                  // ... and everyone's; the stage consumed at s-1 is free again
    {
      const int ahead = s + STAGES - 1;
      int st = stage + STAGES - 1;
      if (st >= STAGES) st -= STAGES;
      if (ahead < num_slabs) issue(ahead, st);
      cp_async_commit();
    }
    const float* a = sA + stage * T::kAStage;
    const float* b = sB + stage * T::kBStage;
    // Fragments are fetched one step ahead of the FFMAs that use them: B (and a K-major A) per step into
    // the other half of bv / av; a pair-major A per k pair, eight floats per quad of rows holding both k.
    // Each step's 64 FFMAs run in a zigzag over stripes of two rows, so that every FFMA shares one
    // register operand with its predecessor, alternately the B and the A value (a0b0 a1b0 a1b1 a0b1 ...).
    float av[2][TM][T::kPair ? 2 : 1], bv[2][TN];
    auto fetch_b = [&](int kk, int h) {
#pragma unroll
      for (int q = 0; q < TN / 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(&b[kk * T::kBRow + (q * T::kThreadsN + tn) * 4]);
        bv[h][q * 4 + 0] = t.x; bv[h][q * 4 + 1] = t.y; bv[h][q * 4 + 2] = t.z; bv[h][q * 4 + 3] = t.w;
      }
    };
    auto fetch_a = [&](int kk, int h) {      // K-major: step kk; pair-major: the pair starting at even kk
#pragma unroll
      for (int q = 0; q < TM / 4; ++q) {
        if (T::kPair) {
          const float* src = &a[((kk >> 1) * T::kARowP + (q * T::kThreadsM + tm) * 4) * 2];
          const float4 t0 = *reinterpret_cast<const float4*>(src);
          const float4 t1 = *reinterpret_cast<const float4*>(src + 4);
          av[h][q * 4 + 0][0] = t0.x; av[h][q * 4 + 0][T::kPair] = t0.y;
          av[h][q * 4 + 1][0] = t0.z; av[h][q * 4 + 1][T::kPair] = t0.w;
          av[h][q * 4 + 2][0] = t1.x; av[h][q * 4 + 2][T::kPair] = t1.y;
          av[h][q * 4 + 3][0] = t1.z; av[h][q * 4 + 3][T::kPair] = t1.w;
        } else {
          const float4 t = *reinterpret_cast<const float4*>(&a[kk * T::kARow + (q * T::kThreadsM + tm) * 4]);
          av[h][q * 4 + 0][0] = t.x; av[h][q * 4 + 1][0] = t.y; av[h][q * 4 + 2][0] = t.z; av[h][q * 4 + 3][0] = t.w;
        }
      }
    };
    fetch_a(0, 0);
    fetch_b(0, 0);
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      if (T::kPair) {
        if (kk + 1 < BK) fetch_b(kk + 1, (kk + 1) & 1);
        if ((kk & 1) == 0 && kk + 2 < BK) fetch_a(kk + 2, ((kk >> 1) + 1) & 1);
      } else if (kk + 1 < BK) {
        fetch_a(kk + 1, (kk + 1) & 1);
        fetch_b(kk + 1, (kk + 1) & 1);
      }
      const int ha = T::kPair ? (kk >> 1) & 1 : kk & 1, ka = T::kPair ? kk & 1 : 0, hb = kk & 1;
#pragma unroll
      for (int i2 = 0; i2 < TM; i2 += 2)
#pragma unroll
        for (int jj = 0; jj < TN; ++jj) {
          const int j = (i2 & 2) ? TN - 1 - jj : jj;
          const int ia = i2 + (jj & 1), ib = i2 + 1 - (jj & 1);
          acc[ia][j] = fmaf(av[ha][ia][ka], bv[hb][j], acc[ia][j]);
          acc[ib][j] = fmaf(av[ha][ib][ka], bv[hb][j], acc[ib][j]);
        }
    }
    if (++stage == STAGES) stage = 0;
  }
  cp_async_wait<0>();

#pragma unroll
  for (int qi = 0; qi < TM / 4; ++qi)
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) {
      const int gm = m0 + row_of(qi * 4 + ii);
      if (gm >= M) continue;
#pragma unroll
      for (int qj = 0; qj < TN / 4; ++qj) {
        const int gn = n0 + (qj * T::kThreadsN + tn) * 4;
        float* p = C + (int64_t)gm * ldc + gn;
        const float* r = &acc[qi * 4 + ii][qj * 4];
        if (gn + 3 < N) *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
        else {
          if (gn + 0 < N) p[0] = r[0];
          if (gn + 1 < N) p[1] = r[1];
          if (gn + 2 < N) p[2] = r[2];
        }
      }
    }
}

template <int BM, int BN, int BK, int TM, int TN, int STAGES, int MIN_CTAS>
static cudaError_t launch_sgemm_pipe(const float* A, int64_t lda, bool trans_a, const float* B, int64_t ldb, float* C,
                                     int64_t ldc, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (trans_a) {
    using T = SgemmPipeTraits<BM, BN, BK, TM, TN, STAGES, true>;
    auto kern = sgemm_f32_pipe_kernel<BM, BN, BK, TM, TN, STAGES, true, MIN_CTAS>;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
      if (e != cudaSuccess) return e;
      attr_dev = dev;
    }
    kern<<<grid, T::kThreads, T::kSmemBytes, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
  } else {
    using T = SgemmPipeTraits<BM, BN, BK, TM, TN, STAGES, false>;
    auto kern = sgemm_f32_pipe_kernel<BM, BN, BK, TM, TN, STAGES, false, MIN_CTAS>;
    static thread_local int attr_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_dev != dev) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes);
      if (e != cudaSuccess) return e;
      attr_dev = dev;
    }
    kern<<<grid, T::kThreads, T::kSmemBytes, stream>>>(A, lda, B, ldb, C, ldc, M, N, K);
  }
  return cudaSuccess;
}

// stages == 2: register-staged double buffer (any alignment); stages >= 3: cp.async ring (16-byte-aligned operands,
// otherwise the launch falls back to the register-staged kernel of the same tile)
struct SgemmCfg { int bm, bn, bk, tm, tn, stages; };
static const SgemmCfg kSgemmCfgs[] = {
    {128, 128, 16, 8, 8, 4}, {128, 128, 32, 8, 8, 3}, {128, 64, 16, 8, 4, 4}, {128, 64, 32, 8, 4, 3},
    {64, 128, 16, 4, 8, 4},
    {128, 128, 16, 8, 8, 2}, {128, 64, 16, 8, 4, 2}, {64, 128, 16, 4, 8, 2}, {64, 64, 16, 4, 4, 2}, {32, 64, 16, 4, 4, 2},
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
  out->stages = kSgemmCfgs[idx].stages;
  out->cta_group = 1;
  out->split_k = 1;
}

// Relative FFMA-issue efficiency of each configuration when the machine is full (measured on large
// squares), used to rank configurations by ceil(tiles / resident CTAs) * tile work / efficiency.
static double sgemm_cfg_rate(const SgemmCfg& c) {
  if (c.stages >= 3) {
    if (c.bm == 128 && c.bn == 128) return c.bk == 32 ? 1.0 : 0.93;
    if (c.bm == 64) return 0.89;
    return c.bk == 32 ? 0.93 : 0.90;
  }
  if (c.bm == 128) return 0.86;
  if (c.bn == 128) return 0.82;
  return 0.72;
}
static int sgemm_cfg_ctas_per_sm(const SgemmCfg& c) {
  if (c.stages >= 3) return 2;
  return (c.bm == 128 && c.bn == 128) ? 2 : (c.bm * c.bn >= 8192 ? 3 : 4);
}

// The configuration with the smallest work on the busiest SM (tiles it runs x tile area / rate); a wave
// holds ctas_per_sm tiles on every SM.
void sgemm_f32_default_config(int M, int N, int sm_count, helix_cfg_t* out) {
  int pick = 0;
  double best = 1e300;
  for (int i = 0; i < kNumSgemmCfgs; ++i) {
    const SgemmCfg& c = kSgemmCfgs[i];
    const int64_t tiles = (int64_t)((M + c.bm - 1) / c.bm) * ((N + c.bn - 1) / c.bn);
    const int per_sm = sgemm_cfg_ctas_per_sm(c);
    const int64_t slots = (int64_t)sm_count * per_sm;
    const int64_t waves = (tiles + slots - 1) / slots;
    // CTAs on the busiest SM over the whole run, in units of tile work
    const int64_t busiest = (waves - 1) * per_sm + ((tiles - (waves - 1) * slots) + sm_count - 1) / sm_count;
    const double t = (double)busiest * c.bm * c.bn / sgemm_cfg_rate(c);
    if (t < best) { best = t; pick = i; }
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
  int bm, bn, bk, stages;
  if (cfg && cfg->tile_m != 0) {
    bm = cfg->tile_m;
    bn = cfg->tile_n;
    bk = cfg->tile_k ? cfg->tile_k : 16;
    stages = cfg->stages ? cfg->stages : 2;
  } else {
    helix_cfg_t def{};
    sgemm_f32_default_config(M, N, sm_count, &def);
    bm = def.tile_m;
    bn = def.tile_n;
    bk = def.tile_k;
    stages = def.stages;
  }
  const bool ta = trans_a != 0;
  if (stages >= 3 && vec) {
    cudaError_t e = cudaErrorInvalidValue;
    if (bm == 128 && bn == 128 && bk == 16) e = launch_sgemm_pipe<128, 128, 16, 8, 8, 4, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 128 && bn == 128 && bk == 8 && stages == 4) e = launch_sgemm_pipe<128, 128, 8, 8, 8, 4, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 128 && bn == 128 && bk == 8) e = launch_sgemm_pipe<128, 128, 8, 8, 8, 3, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 128 && bn == 128 && bk == 32) e = launch_sgemm_pipe<128, 128, 32, 8, 8, 3, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 128 && bn == 64 && bk == 16) e = launch_sgemm_pipe<128, 64, 16, 8, 4, 4, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 128 && bn == 64 && bk == 32) e = launch_sgemm_pipe<128, 64, 32, 8, 4, 3, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else if (bm == 64 && bn == 128 && bk == 16) e = launch_sgemm_pipe<64, 128, 16, 4, 8, 4, 2>(A, lda, ta, B, ldb, C, ldc, M, N, K, stream);
    else return HELIX_ERR_UNSUPPORTED;
    if (e != cudaSuccess) return HELIX_ERR_CUDA;
    ++*launches;
    return cudaGetLastError() == cudaSuccess ? HELIX_OK : HELIX_ERR_CUDA;
  }
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
