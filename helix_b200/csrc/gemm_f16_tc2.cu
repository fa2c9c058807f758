// fp16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with a 256 x BN tile per pair of SMs.
//
// Same contract as the one-CTA kernel in gemm_f16_tc.cu (C[M,N] = A[M,K] * B[N,K]^T, fp32
// accumulate in TMEM, fp16 out) for the large, compute-bound shapes.  Two CTAs of a cluster share
// one output tile: CTA r loads its own 128 rows of A and its own half (BN/2 rows) of the B tile,
// the even CTA issues one MMA per K=16 step for both tensor cores, and each CTA keeps the
// accumulator of its 128 rows in its own TMEM.  Per CTA a K slab is 16 KiB of A plus BN/2 x 128
// bytes of B (32 KiB at BN = 256 against 48 KiB for the one-CTA 128 x 256 tile), so the
// shared-memory ring is 6 deep instead of 4 and each loaded byte feeds 1.5x the math: the TMA
// latency that the 4-stage ring leaves exposed is covered.
//
// Synchronisation (all waits bounded):
//   full[s]   lives in the even CTA; it expects the bytes of BOTH CTAs' loads.  Each CTA's TMA
//             loads name that barrier through its cluster address (no multicast: every CTA fetches
//             only its own boxes).
//   empty[s]  and tmem_full[a] exist in both CTAs and are signalled together by one
//             tcgen05.commit addressed to both CTAs of the pair.
//   tmem_empty[a] lives in the even CTA and counts the 8 epilogue warps of the pair; the odd CTA's
//             warps arrive on it remotely.
#include <cuda.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace helix {

namespace {

constexpr int kBM = 128;   // rows per CTA; the pair covers 256
constexpr int kBK = 64;
constexpr int kATileBytes = kBM * kBK * 2;
constexpr int kPairProducerWarps = 3;   // warp 0 and warps 6, 7 issue TMA loads (slab n: issuer n % load_warps)
constexpr int kThreads = 32 + 32 + 128 + 64;
constexpr int kStagingBytes = 2 * 128 * 128;     // two 128-row x 128-byte boxes shared by the four epilogue warps
constexpr int kEpiBarrier = 1;                   // named barrier of the 128 epilogue threads
constexpr int kTokBarrier2 = 10;                 // named barriers 10, 11: issue order of two MMA warps that alternate K slabs
constexpr int kFwdBarrier2 = 2;                  // named barriers 2..9: arrival of a group of ring stages, forwarded to the MMA warp

struct Gemm2Params {
  __half* C;
  int64_t ldc, stride_c;
  int PM, PN, K, batch;
  int tiles_m, tiles_n, num_kb, total_tiles;  // tiles_m counts 256-row pair tiles
  int raster, stages;
  int load_warps;   // issuing warps per CTA, <= stages (see the one-CTA kernel's producer)
  int tma_store, independent;
  int probe;        // tuning instrument (helix_cfg_t.probe): 1 = issue no MMA, 2 = no A loads, 4 = no B loads
  int dual;         // 1: warps 1 and 7 of the even CTA issue the MMAs of alternate K slabs (needs load_warps <= 2, group 1)
  int group;        // ring stages that share one "full" barrier (one wait of the MMA issuer per group)
  FastDiv fd_grp;
  int* status;
  FastDiv fd_per_batch, fd_group, fd_raster, fd_num_kb;   // reciprocals for the tile decoder
  unsigned long long* trace;                   // optional per-CTA timeline (null = off)
  // stream-K schedule: dp_rounds whole tiles per pair, then the K slabs of the sk_tiles remaining
  // tiles dealt out in ranges of sk_upc slabs (<= num_kb, so a range touches at most two tiles);
  // a pair that computes only part of a tile leaves its fp32 accumulator in a slot of `partial`
  // ([2 * pairs][256][BN]) and a fix-up kernel adds the slots of each such tile in pair order.
  int stream_k, dp_rounds, sk_tiles, sk_upc;
  float* partial;
};

struct Item2 {
  int tile, kb0, kb1;
  int slot;   // < 0: the whole K range, result goes straight to C
};

__device__ __forceinline__ void trace2(const Gemm2Params& p, int word) {
  if (p.trace != nullptr) p.trace[(size_t)blockIdx.x * kTraceWords + word] = (unsigned long long)clock64();
}
__device__ __forceinline__ void trace2_tile(const Gemm2Params& p, int idx, int slot) {
  if (idx < kTraceTiles) trace2(p, 8 + idx * 6 + slot);
}
__device__ __forceinline__ void trace2_slab(const Gemm2Params& p, int which, int n) {
  if (n < kTraceSlabs) trace2(p, 8 + 6 * kTraceTiles + which * kTraceSlabs + n);
}

struct Tile2 {
  int m_blk, n_blk, b;
};

__device__ __forceinline__ Tile2 decode_tile2(const Gemm2Params& p, int t) {
  Tile2 w;
  int r, gid;
  fast_divmod(t, p.fd_per_batch, w.b, r);
  fast_divmod(r, p.fd_group, gid, r);
  const int first_m = gid * p.raster;
  const int gm = min(p.raster, p.tiles_m - first_m);
  const int q = gm == p.raster ? fast_div(r, p.fd_raster) : r / gm;   // plain division in the last group only
  w.m_blk = first_m + (r - q * gm);
  w.n_blk = q;
  return w;
}

// The idx-th work item of a pair; every role of both CTAs walks the same sequence.
__device__ __forceinline__ bool get_item2(const Gemm2Params& p, int pair, int num_pairs, int idx, Item2& it) {
  if (!p.stream_k || idx < p.dp_rounds) {
    it.tile = pair + idx * num_pairs;
    it.kb0 = 0;
    it.kb1 = p.num_kb;
    it.slot = -1;
    return p.stream_k || it.tile < p.total_tiles;
  }
  const int s = idx - p.dp_rounds;   // first / second tile the pair's slab range touches
  if (s > 1) return false;
  const int sk_units = p.sk_tiles * p.num_kb;
  const int u0 = min(sk_units, pair * p.sk_upc);
  const int u1 = min(sk_units, u0 + p.sk_upc);
  if (u0 >= u1) return false;
  const int j0 = fast_div(u0, p.fd_num_kb);
  const int split = min(u1, (j0 + 1) * p.num_kb);
  int j, a, b;
  if (s == 0) { j = j0; a = u0; b = split; }
  else { j = j0 + 1; a = split; b = u1; }
  if (a >= b) return false;
  it.tile = p.dp_rounds * num_pairs + j;
  it.kb0 = a - j * p.num_kb;
  it.kb1 = b - j * p.num_kb;
  it.slot = (it.kb0 == 0 && it.kb1 == p.num_kb) ? -1 : 2 * pair + s;
  return true;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier that may live in the other CTA of the pair.  The arrival only has to order
// this thread's TMEM reads (tcgen05.fence::before_thread_sync precedes it), so it carries the
// default CTA-scope semantics: a cluster-scope release was measured to hold the thread for about
// a microsecond per tile.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are credited to a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const void* desc, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, "
      "%5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(desc)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(NCOLS)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int NCOLS>
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(NCOLS) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair, once every
// MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint32_t mask = 3;
  asm volatile(
      "{\n\t.reg .b16 lo, hi;\n\t"
      "mov.b32 {lo, hi}, %1;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], lo;\n\t}" ::"r"(
          smem_u32(bar)),
      "r"(mask)
      : "memory");
}

// The same two instructions for a warp that walks its issue loop convergently: every lane executes the statement,
// one elected lane issues (see umma_f16_ss_elect in common.cuh).
__device__ __forceinline__ void umma_f16_ss_pair_elect(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                       bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@q tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair_elect(uint64_t* bar) {
  const uint32_t mask = 3;
  asm volatile(
      "{\n\t.reg .b16 lo, hi;\n\t.reg .pred q;\n\t"
      "mov.b32 {lo, hi}, %1;\n\t"
      "elect.sync _|q, 0xffffffff;\n\t"
      "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], lo;\n\t}" ::"r"(
          smem_u32(bar)),
      "r"(mask)
      : "memory");
}

// Dual issue (the default; probe bit 9 turns it off): two warps of the even CTA walk this loop and issue the MMAs of alternate K slabs
// (slab n belongs to warp n & 1 = ME).  Each waits for its own slabs' arrival barrier itself (one barrier per stage):
// the ~200 cycles a shared-memory read spends behind the warp's own queued MMAs, its descriptors and its commit all
// run while the other warp's four MMAs of 128 pipe cycles each are being issued.  The order of the MMAs is fixed by
// a token: the owner of slab n - 1 arrives at a named barrier after issuing, fenced, and the owner of slab n meets
// it there before issuing, so the accumulation order -- every bit of the result -- is that of one issuer.  Both
// warps walk the whole sequence whatever happens (after a failed wait nothing is issued, the rendezvous are kept).
template <int BN, int ME>
__device__ __forceinline__ void pair_dual_issue_loop(const Gemm2Params& p, const int pair, const int num_pairs,
                                                     const int lane, const int stages, uint8_t* sA, uint8_t* sB,
                                                     uint64_t* full_bar, uint64_t* empty_bar, uint64_t* tmem_full,
                                                     uint64_t* tmem_empty, volatile int* abort_flag,
                                                     const uint32_t tmem_base) {
  constexpr int kBHalfBytes = (BN / 2) * kBK * 2;
  constexpr uint32_t kIdesc = umma_idesc_f16(2 * kBM, BN);
  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  int nslab = 0;
  Item2 it;
  for (int idx = 0; get_item2(p, pair, num_pairs, idx, it); ++idx) {
    const int acc = idx & 1;
    const uint32_t acc_phase = (idx >> 1) & 1;
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status));
    tc_fence_after_sync();
    if (lane == 0 && ME == 0) trace2_tile(p, idx, 2);
    const uint32_t d_tmem = tmem_base + acc * BN;
    for (int kb = it.kb0; kb < it.kb1; ++kb) {
      const int n = nslab++;
      if ((n & 1) == ME) {
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status));
        if (lane == 0) trace2_slab(p, 1, n);
        tc_fence_after_sync();
        const uint64_t da = umma_desc_sw128(smem_u32(sA + (size_t)stage * kATileBytes));
        const uint64_t db = umma_desc_sw128(smem_u32(sB + (size_t)stage * kBHalfBytes));
        if (n > 0) {
          named_bar_sync(kTokBarrier2 + ((n - 1) & 1), 64);
          tc_fence_after_sync();
        }
        if (ok && !(p.probe & 1)) {
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_f16_ss_pair_elect(d_tmem, da + 2 * k, db + 2 * k, kIdesc, (kb > it.kb0) || (k > 0));
        }
        tc_fence_before_sync();
        asm volatile("bar.arrive %0, 64;" ::"r"(kTokBarrier2 + (n & 1)) : "memory");
        if (ok) umma_commit_pair_elect(&empty_bar[stage]);
      }
      if (++stage == stages) { stage = 0; phase ^= 1; }
    }
    if (ok) umma_commit_pair_elect(&tmem_full[acc]);   // both warps, each for its own MMAs (barrier count 2)
    if (lane == 0 && ME == 0) trace2_tile(p, idx, 3);
  }
  // the token of the last slab is met by the warp that did not issue it, so that no arrival is left over
  if (nslab > 0 && ((nslab - 1) & 1) != ME) named_bar_sync(kTokBarrier2 + ((nslab - 1) & 1), 64);
}

template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_f16_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const Gemm2Params p) {
  constexpr int kBHalfBytes = (BN / 2) * kBK * 2;
  constexpr int kStageBytes = kATileBytes + kBHalfBytes;
  constexpr int kTmemCols = 2 * BN <= 256 ? 256 : 512;
  constexpr uint32_t kIdesc = umma_idesc_f16(2 * kBM, BN);

  griddep_launch_dependents();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  uint8_t* sA = smem;
  uint8_t* sB = smem + (size_t)stages * kATileBytes;
  uint8_t* sC = smem + (size_t)stages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sC + kStagingBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + 8;
  uint64_t* tmem_full = bars + 16;
  uint64_t* tmem_empty = bars + 18;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    if (p.trace != nullptr) {
      p.trace[(size_t)blockIdx.x * kTraceWords + 0] = global_timer_ns();
      trace2(p, 1);
    }
    for (int s = 0; s < stages; ++s) {
      if (s * p.group < stages) mbar_init(&full_bar[s], p.group);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], p.dual ? 2 : 1);
      mbar_init(&tmem_empty[a], 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.tma_store) tma_prefetch_desc(&tmap_c);
  }
  if (warp == 1) tmem_alloc_pair<kTmemCols>(tmem_ptr_smem);
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers exist before anything is signalled across the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (!p.independent) griddep_wait();
  if (threadIdx.x == 0) trace2(p, 2);

  if (warp == 0 || warp >= 6) {
    // ------------------------------------------------------------------ TMA producers (each CTA)
    // Issuer j requests the slabs n = j, j + load_warps, ... of the CTA's slab sequence; slab n
    // lives in ring stage n % stages.  One thread cannot keep the ring full: a tensor copy holds
    // its issuing thread for a few hundred cycles.
    const int issuer = warp == 0 ? 0 : warp - 5;
    // With at most two issuing warps, warp 7 of the even CTA watches the ring's arrival barriers for the MMA warp
    // and meets it at a named barrier per group of stages: a shared-memory read by the MMA warp itself would queue
    // behind the MMAs it has just issued.  Both warps walk the same sequence of groups to its end whatever
    // happens (after a failed wait only the rendezvous are kept), in lockstep per group.
    if (p.dual) {
      if (warp == 7 && rank == 0)   // second MMA-issuing warp (it issues no loads: load_warps <= 2)
        pair_dual_issue_loop<BN, 1>(p, pair, num_pairs, lane, stages, sA, sB, full_bar, empty_bar, tmem_full, tmem_empty,
                                    abort_flag, tmem_base);
    } else if (warp == 7 && rank == 0 && p.load_warps < kPairProducerWarps) {
      bool ok = true;
      int stage = 0, gpos = 0, gidx = 0;
      uint32_t phase = 0;
      Item2 it;
      for (int idx = 0; get_item2(p, pair, num_pairs, idx, it); ++idx) {
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (gpos == 0) {
            if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[gidx], phase, abort_flag, p.status));
            named_bar_sync(kFwdBarrier2 + gidx, 64);
          }
          if (++gpos == p.group) { gpos = 0; ++gidx; }
          if (++stage == stages) { stage = 0; phase ^= 1; gidx = 0; }
        }
      }
    }
    if (lane == 0 && issuer < p.load_warps) {
      bool ok = true;
      int n_start = 0;
      int my_n = issuer;     // next slab this issuer requests; stage and use parity follow it
      int stage = issuer;    // load_warps <= stages
      uint32_t phase = 0;
      Item2 it;
      for (int tidx = 0; ok && get_item2(p, pair, num_pairs, tidx, it); ++tidx) {
        const Tile2 w = decode_tile2(p, it.tile);
        const int nkb = it.kb1 - it.kb0;
        if (issuer == 0) trace2_tile(p, tidx, 0);
        for (; my_n < n_start + nkb; my_n += p.load_warps) {
          const int kb = it.kb0 + (my_n - n_start);
          ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
          if (!ok) break;
          trace2_slab(p, 0, my_n);
          const bool load_a = !(p.probe & 2), load_b = !(p.probe & 4);
          uint64_t* const fb = &full_bar[fast_div(stage, p.fd_grp)];
          if (rank == 0) {
            if (load_a || load_b)
              mbar_arrive_expect_tx(fb, 2 * ((load_a ? kATileBytes : 0) + (load_b ? kBHalfBytes : 0)));
            else
              mbar_arrive(fb);
          }
          const uint32_t full_leader = map_to_cta(smem_u32(fb), 0);
          if (load_a)
            tma_load_3d_pair(sA + (size_t)stage * kATileBytes, &tmap_a, full_leader, kb * kBK,
                             w.m_blk * 2 * kBM + (int)rank * kBM, w.b);
          if (load_b)
            tma_load_3d_pair(sB + (size_t)stage * kBHalfBytes, &tmap_b, full_leader, kb * kBK,
                             w.n_blk * BN + (int)rank * (BN / 2), w.b);
          stage += p.load_warps;
          if (stage >= stages) { stage -= stages; phase ^= 1; }
        }
        n_start += nkb;
        if (issuer == 0) trace2_tile(p, tidx, 1);
      }
      // a short last group of the pair's slab sequence is completed by plain arrivals (even CTA: the
      // barriers live there), each ordered after the release of its ring stage like a real slab
      const int n_pad = (n_start + p.group - 1) / p.group * p.group;
      for (; ok && my_n < n_pad; my_n += p.load_warps) {
        ok = mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status);
        if (!ok) break;
        if (rank == 0) mbar_arrive(&full_bar[fast_div(stage, p.fd_grp)]);
        stage += p.load_warps;
        if (stage >= stages) { stage -= stages; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    // The whole warp walks the loop convergently (warp-uniform state, waits end in a vote) and one elected lane
    // issues.  With a watcher warp (forward) the arrival of a group of stages comes through a named barrier and the
    // sequence is walked to its end even after a failed wait (ok = false: only the rendezvous are kept).
    if (rank == 0 && p.dual) {
      pair_dual_issue_loop<BN, 0>(p, pair, num_pairs, lane, stages, sA, sB, full_bar, empty_bar, tmem_full, tmem_empty,
                                  abort_flag, tmem_base);
    } else if (rank == 0) {
      const bool forward = p.load_warps < kPairProducerWarps;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int nslab = 0;
      int gpos = 0, gidx = 0;   // position of the next slab inside its group of stages, and the group
      Item2 it;
      for (int idx = 0; (forward || ok) && get_item2(p, pair, num_pairs, idx, it); ++idx) {
        const int acc = idx & 1;
        const uint32_t acc_phase = (idx >> 1) & 1;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status));
        if (!ok && !forward) break;
        tc_fence_after_sync();
        if (lane == 0) trace2_tile(p, idx, 2);
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          // one rendezvous (or wait) per group of stages; the stages are still released one by one
          if (gpos == 0) {
            if (forward) {
              named_bar_sync(kFwdBarrier2 + gidx, 64);
            } else {
              ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[gidx], phase, abort_flag, p.status));
              if (!ok) break;
            }
          }
          if (++gpos == p.group) { gpos = 0; ++gidx; }
          if (lane == 0) trace2_slab(p, 1, nslab);
          ++nslab;
          tc_fence_after_sync();
          const uint64_t da = umma_desc_sw128(smem_u32(sA + (size_t)stage * kATileBytes));
          const uint64_t db = umma_desc_sw128(smem_u32(sB + (size_t)stage * kBHalfBytes));
          if (ok && !(p.probe & 1)) {
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_f16_ss_pair_elect(d_tmem, da + 2 * k, db + 2 * k, kIdesc, (kb > it.kb0) || (k > 0));
          }
          if (ok) umma_commit_pair_elect(&empty_bar[stage]);
          if (++stage == stages) { stage = 0; phase ^= 1; gidx = 0; }
        }
        if (ok) umma_commit_pair_elect(&tmem_full[acc]);
        if (lane == 0) trace2_tile(p, idx, 3);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (each CTA: its 128 rows)
    const int quarter = warp & 3;
    bool ok = true;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) && ((p.stride_c & 7) == 0);
    int box = 0;   // staging box in use; alternates over the whole run of the warp, across tiles
    Item2 it;
    for (int idx = 0; ok && get_item2(p, pair, num_pairs, idx, it); ++idx) {
      const Tile2 w = decode_tile2(p, it.tile);
      const int acc = idx & 1;
      const uint32_t acc_phase = (idx >> 1) & 1;
      ok = mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status);
      ok = named_bar_and(kEpiBarrier, 128, ok);   // the four warps go on, or give up, together
      if (!ok) break;
      tc_fence_after_sync();
      if (quarter == 0 && lane == 0) trace2_tile(p, idx, 4);
      const int cta_row0 = w.m_blk * 2 * kBM + (int)rank * kBM;
      const int row0 = cta_row0 + quarter * 32;
      const int row = row0 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      if (it.slot >= 0) {
        // part of a tile's K range: the fp32 accumulator (padding included) goes to this pair's slot of
        // 256 x BN floats, stored lane-major (the four floats (row, 4j..4j+3) of a warp's 32 rows side by side),
        // so that every store of a warp covers 512 contiguous bytes
        float* dst = p.partial + (size_t)it.slot * (2 * kBM) * BN +
                     ((size_t)(rank * 4 + quarter) * (BN / 4) * 32 + lane) * 4;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < 32; jj += 4)
            *reinterpret_cast<float4*>(dst + (size_t)((c0 + jj) / 4) * 128) =
                make_float4(__uint_as_float(r[jj]), __uint_as_float(r[jj + 1]), __uint_as_float(r[jj + 2]),
                            __uint_as_float(r[jj + 3]));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
        if (quarter == 0 && lane == 0) trace2_tile(p, idx, 5);
        continue;
      }
      uint32_t ra[32], rb[32], na[32], nb[32];
      // 64 columns at a time: the four warps put their 32 rows each into one 128-row staging box
      // and one thread sends the box with a single TMA store (issuing a tensor copy holds its
      // thread for a few hundred cycles, so one 16 KiB store per chunk instead of four 4 KiB ones);
      // two boxes alternate so that a store drains while the next box is filled.
      auto emit = [&](const uint32_t (&lo)[32], const uint32_t (&hi)[32], int c0) {
        const int col0 = w.n_blk * BN + c0;
        if (col0 >= p.PN || cta_row0 >= p.PM) return;   // uniform over the four warps: nothing but padding
        if (p.tma_store) {
          uint8_t* stage_box = sC + box * (128 * 128);
          const uint32_t row_base = smem_u32(stage_box) + (quarter * 32 + lane) * 128;
          box ^= 1;
          if (quarter == 0 && lane == 0) tma_store_wait_read_1();   // the store issued two boxes ago has left this buffer
          named_bar_sync(kEpiBarrier, 128);
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            const uint32_t* src = ch < 4 ? &lo[ch * 8] : &hi[(ch - 4) * 8];
            __half2 h0 = __floats2half2_rn(__uint_as_float(src[0]), __uint_as_float(src[1]));
            __half2 h1 = __floats2half2_rn(__uint_as_float(src[2]), __uint_as_float(src[3]));
            __half2 h2 = __floats2half2_rn(__uint_as_float(src[4]), __uint_as_float(src[5]));
            __half2 h3 = __floats2half2_rn(__uint_as_float(src[6]), __uint_as_float(src[7]));
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_base + ((ch ^ (lane & 7)) << 4)),
                         "r"(*reinterpret_cast<uint32_t*>(&h0)), "r"(*reinterpret_cast<uint32_t*>(&h1)),
                         "r"(*reinterpret_cast<uint32_t*>(&h2)), "r"(*reinterpret_cast<uint32_t*>(&h3))
                         : "memory");
          }
          fence_proxy_async_smem();
          named_bar_sync(kEpiBarrier, 128);
          if (quarter == 0 && lane == 0) {
            tma_store_3d(&tmap_c, stage_box, col0, cta_row0, w.b);
            tma_store_commit();
          }
        } else if (row < p.PM) {
          __half* dst = p.C + (int64_t)w.b * p.stride_c + (int64_t)row * p.ldc + col0;
#pragma unroll
          for (int jj = 0; jj < 64; jj += 8) {
            const uint32_t* src = jj < 32 ? &lo[jj] : &hi[jj - 32];
            if (vec_ok && col0 + jj + 8 <= p.PN) {
              uint4 v;
              __half2 h0 = __floats2half2_rn(__uint_as_float(src[0]), __uint_as_float(src[1]));
              __half2 h1 = __floats2half2_rn(__uint_as_float(src[2]), __uint_as_float(src[3]));
              __half2 h2 = __floats2half2_rn(__uint_as_float(src[4]), __uint_as_float(src[5]));
              __half2 h3 = __floats2half2_rn(__uint_as_float(src[6]), __uint_as_float(src[7]));
              v.x = *reinterpret_cast<uint32_t*>(&h0);
              v.y = *reinterpret_cast<uint32_t*>(&h1);
              v.z = *reinterpret_cast<uint32_t*>(&h2);
              v.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(dst + jj) = v;
            } else {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (col0 + jj + q < p.PN) dst[jj + q] = __float2half_rn(__uint_as_float(src[q]));
            }
          }
        }
      };
      tmem_ld_32x32b_x32(taddr, ra);
      tmem_ld_32x32b_x32(taddr + 32, rb);
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 128) {
        tmem_ld_wait();
        if (c0 + 64 < BN) {
          tmem_ld_32x32b_x32(taddr + c0 + 64, na);
          tmem_ld_32x32b_x32(taddr + c0 + 96, nb);
        }
        emit(ra, rb, c0);
        if (c0 + 64 < BN) {
          tmem_ld_wait();
          if (c0 + 128 < BN) {
            tmem_ld_32x32b_x32(taddr + c0 + 128, ra);
            tmem_ld_32x32b_x32(taddr + c0 + 160, rb);
          }
          emit(na, nb, c0 + 64);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty[acc]), 0));
      if (quarter == 0 && lane == 0) trace2_tile(p, idx, 5);
    }
    // the staging boxes must have been read before the CTA's shared memory goes away; the writes
    // themselves complete with the grid
    if (p.tma_store && quarter == 0 && lane == 0) tma_store_wait_read();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();   // nothing of the pair still refers to this CTA's barriers or shared memory
  // A launch that did not wait for its predecessor before its work waits for it now, after its last
  // store: the kernel then cannot complete before everything queued ahead of it has, so completion
  // order along the stream stays transitive for whatever is queued next.
  if (p.independent) griddep_wait();
  if (threadIdx.x == 0 && p.trace != nullptr) {
    trace2(p, 3);
    p.trace[(size_t)blockIdx.x * kTraceWords + 4] = global_timer_ns();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_pair<kTmemCols>(tmem_base);
  }
}

// Stream-K fix-up for pair tiles: a dealt-out tile whose K slabs were shared by several pairs is the
// sum of their fp32 slots, added in pair order (deterministic) and rounded once.  Grid: (blocks per
// tile, dealt-out tiles); one thread per four consecutive columns of a tile row.
__global__ void gemm2_streamk_fixup_kernel(const Gemm2Params p, int bn, int num_pairs) {
  const int j = blockIdx.y;
  const int u_lo = j * p.num_kb, u_hi = (j + 1) * p.num_kb;
  const int c_lo = u_lo / p.sk_upc, c_hi = (u_hi - 1) / p.sk_upc;
  if (c_lo == c_hi) return;   // computed whole by one pair and already stored
  const int quad = blockIdx.x * blockDim.x + threadIdx.x;
  const int quads_per_row = bn >> 2;
  if (quad >= 2 * kBM * quads_per_row) return;
  const int trow = quad / quads_per_row, tcol = (quad - trow * quads_per_row) << 2;
  const Tile2 w = decode_tile2(p, p.dp_rounds * num_pairs + j);
  const int row = w.m_blk * 2 * kBM + trow, col = w.n_blk * bn + tcol;
  if (row >= p.PM || col >= p.PN) return;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c = c_lo; c <= c_hi; ++c) {
    const int first_tile = (c * p.sk_upc) / p.num_kb;
    const int slot = 2 * c + (j == first_tile ? 0 : 1);
    const float4 v = *reinterpret_cast<const float4*>(
        p.partial + (size_t)slot * (2 * kBM) * bn + ((size_t)((trow >> 5) * (bn >> 2) + (tcol >> 2)) * 32 + (trow & 31)) * 4);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  const float vals[4] = {s.x, s.y, s.z, s.w};
  __half* dst = p.C + (int64_t)w.b * p.stride_c + (int64_t)row * p.ldc + col;
  if (col + 3 < p.PN && (p.ldc & 3) == 0 && (p.stride_c & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 7) == 0) {
    __half2 h0 = __floats2half2_rn(vals[0], vals[1]);
    __half2 h1 = __floats2half2_rn(vals[2], vals[3]);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&h0);
    pk.y = *reinterpret_cast<uint32_t*>(&h1);
    *reinterpret_cast<uint2*>(dst) = pk;
  } else {
    for (int q = 0; q < 4; ++q)
      if (col + q < p.PN) dst[q] = __float2half_rn(vals[q]);
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

int make_map(CUtensorMap* map, const void* base, int64_t inner, int64_t rows, int64_t batch, int64_t ld, int64_t bs,
             int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return HELIX_ERR_CUDA;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 7) || (batch > 1 && (bs & 7))) return HELIX_ERR_ALIGN;
  if (batch <= 1) bs = rows * ld;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)std::max<int64_t>(batch, 1)};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HELIX_OK : HELIX_ERR_CUDA;
}

template <int BN>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const Gemm2Params& p,
                        int grid, size_t smem, cudaStream_t stream) {
  auto kern = gemm_f16_tc2_kernel<BN>;
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
  cudaError_t e = cudaLaunchKernelEx(&lc, kern, ta, tb, tc, p);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    kern<<<grid, kThreads, smem, stream>>>(ta, tb, tc, p);
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace

int gemm_f16_pair_max_stages(int bn) {
  const int budget = 227 * 1024 - 1024 - 256 - kStagingBytes;
  return std::min(8, budget / (kATileBytes + (bn / 2) * kBK * 2));
}

// Workspace of the stream-K schedule on CTA pairs: two fp32 slots of 256 x BN per pair.
size_t gemm_f16_pair_workspace_bytes(const helix_cfg_t& cfg, int M, int N, int K, int batch, int sm_count) {
  if (!cfg.stream_k) return 0;
  const int bn = cfg.tile_n;
  const int64_t tiles = (int64_t)((M + 2 * kBM - 1) / (2 * kBM)) * ((N + bn - 1) / bn) * std::max(batch, 1);
  const int pairs = std::max(1, sm_count / 2);
  if (tiles % pairs == 0 || (K + kBK - 1) / kBK < 2) return 0;
  return (size_t)2 * pairs * 2 * kBM * bn * sizeof(float);
}

// cta_group = 2 configurations: 256 x BN tiles round-robin over CTA pairs; with stream_k the K
// slabs of the tiles beyond the last whole round are dealt evenly to all pairs.
int gemm_f16_pair_launch(const helix_cfg_t& cfg, const void* A, int64_t lda, const void* B, int64_t ldb, void* C,
                         int64_t ldc, int M, int N, int K, int batch, int64_t sa, int64_t sb, int64_t sc, void* ws,
                         size_t ws_bytes, int* status_dev, int sm_count, bool independent, cudaStream_t stream,
                         int64_t* launches) {
  const int bn = cfg.tile_n;
  if (bn != 256 && bn != 192 && bn != 128) return HELIX_ERR_UNSUPPORTED;
  if (cfg.swap_ab || cfg.split_k > 1) return HELIX_ERR_UNSUPPORTED;
  Gemm2Params p{};
  p.PM = M; p.PN = N; p.K = K; p.batch = batch;
  p.C = static_cast<__half*>(C);
  p.ldc = ldc; p.stride_c = sc;
  p.status = status_dev;
  p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  p.tiles_n = (N + bn - 1) / bn;
  p.num_kb = (K + kBK - 1) / kBK;
  const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n * batch;
  if (tiles <= 0 || tiles > 0x3fffffff) return HELIX_ERR_INVALID;
  p.total_tiles = (int)tiles;
  p.raster = cfg.raster > 0 ? cfg.raster : 8;
  const int smax = gemm_f16_pair_max_stages(bn);
  p.stages = cfg.stages > 0 ? std::min(cfg.stages, smax) : smax;
  if (p.stages < 2) return HELIX_ERR_UNSUPPORTED;
  // measured with the forwarded arrivals (microseconds at 1 / 2 / 3 stages per group): 4096^3 104.6 / 102.0 / 108.5,
  // 8192 x 768 x 3072 36.7 / 35.3 / 38.1, 8192 x 2304 x 768 23.8 / 23.6 / 24.1
  p.group = p.stages >= 4 ? 2 : 1;
  // Two issuing warps, each waiting for its own slabs (one arrival barrier per stage), unless probe bit 9 asks for
  // the single issuer or a third loading warp needs warp 7.  Measured against the single issuer with two stages per
  // group (microseconds): 4096^3 101.7 -> 101.0, 8192 x 2304 x 768 23.9 -> 23.0, 8192 x 3072 x 768 32.3 -> 31.0,
  // 8192^3 and 2048 x 14336 x 4096 within 1 %; on 128-wide pair tiles 12-20 % (4096^3 137.7 -> 122.6).
  p.dual = (!(cfg.probe & 0x200) && (cfg.load_group > 0 ? cfg.load_group : 2) <= 2) ? 1 : 0;
  if ((cfg.probe >> 4) & 7) p.group = (cfg.probe >> 4) & 7;   // tuning override
  if (p.dual) p.group = 1;
  while (p.group > 1 && p.stages / p.group < 2) --p.group;
  p.stages = p.stages / p.group * p.group;
  p.fd_grp = make_fastdiv(p.group);
  p.load_warps = std::max(1, std::min({cfg.load_group > 0 ? cfg.load_group : 2, kPairProducerWarps, p.stages}));
  p.fd_per_batch = make_fastdiv(p.tiles_m * p.tiles_n);
  p.fd_group = make_fastdiv(p.raster * p.tiles_n);
  p.fd_raster = make_fastdiv(p.raster);
  p.fd_num_kb = make_fastdiv(p.num_kb);
  int pairs = (int)std::min<int64_t>(tiles, sm_count / 2);
  bool fixup = false;
  if (cfg.stream_k && p.num_kb >= 2 && sm_count >= 2 && tiles % (sm_count / 2) != 0) {
    pairs = sm_count / 2;
    p.stream_k = 1;
    p.dp_rounds = (int)(tiles / pairs);
    p.sk_tiles = (int)(tiles - (int64_t)p.dp_rounds * pairs);
    const int64_t units = (int64_t)p.sk_tiles * p.num_kb;
    int upc = (int)((units + pairs - 1) / pairs);
    upc = std::max(upc, std::min(4, p.num_kb));   // no slivers; still <= num_kb because sk_tiles < pairs
    p.sk_upc = std::max(1, upc);
    const size_t need = (size_t)2 * pairs * 2 * kBM * bn * sizeof(float);
    if (!ws || ws_bytes < need) return HELIX_ERR_WORKSPACE;
    p.partial = static_cast<float*>(ws);
    fixup = true;
  }
  p.trace = gemm_f16_trace_for_grid(2 * pairs);
  p.probe = cfg.probe & 7;
  // a launch that shares its workspace with its neighbours on the stream is never independent of them
  p.independent = (independent && !fixup) ? 1 : 0;
  CUtensorMap ta, tb, tc;
  int rc;
  if ((rc = make_map(&ta, A, K, M, batch, lda, sa, kBM)) != HELIX_OK) return rc;
  if ((rc = make_map(&tb, B, K, N, batch, ldb, sb, bn / 2)) != HELIX_OK) return rc;
  tc = tb;
  p.tma_store = 0;
  if ((ldc & 7) == 0 && (sc & 7) == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0 &&
      make_map(&tc, C, N, M, batch, ldc, sc, kBM) == HELIX_OK)
    p.tma_store = 1;
  const size_t smem = 1024 + (size_t)p.stages * (kATileBytes + (bn / 2) * kBK * 2) + kStagingBytes + 256;
  const cudaError_t e = bn == 256   ? launch_pair<256>(ta, tb, tc, p, 2 * pairs, smem, stream)
                        : bn == 192 ? launch_pair<192>(ta, tb, tc, p, 2 * pairs, smem, stream)
                                    : launch_pair<128>(ta, tb, tc, p, 2 * pairs, smem, stream);
  if (e != cudaSuccess) return HELIX_ERR_CUDA;
  ++*launches;
  if (fixup) {
    const dim3 fgrid((2 * kBM * (bn >> 2) + 255) / 256, p.sk_tiles);
    gemm2_streamk_fixup_kernel<<<fgrid, 256, 0, stream>>>(p, bn, pairs);
    if (cudaGetLastError() != cudaSuccess) return HELIX_ERR_CUDA;
    ++*launches;
  }
  return HELIX_OK;
}

}  // namespace helix
