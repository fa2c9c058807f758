"""Search space, profiled dictionary and cost model for the sm_100a kernels.

The reference profiles every tile configuration once on a one-CTA problem and
predicts ``ceil(blocks / 108) * t_cfg`` with K ignored (scripts/Ampere_FP16/
Ampere_FP16_gemm.py:420-430, profile_Ampere_FP16.py:17-62).  The same idea, re-derived
for a persistent tcgen05 kernel:

* a configuration is (stages, tile_m, tile_n, cta_group, swap_ab, mode) with mode 0 = whole
  tiles round-robin, 1 = stream-K, 2..4 = split-K over that many slices summed by the last-arriving
  CTA; GEMV configurations start with 0 like the reference's (0, 1, 128, 0, 0, splitK) keys:
  (0, 1, rows_per_warp, loads_in_flight, 0, split_k);
* each GEMM tile width is probed at two K values on a full-machine problem, which gives a
  fixed cost per launch and a cost per 64-deep K slab (the reference's single number per
  configuration cannot separate the two, so its model drops K);
* the time of a shape is  t_fixed + slabs_per_CTA * t_slab,  slabs counted from the wave
  structure on the queried SM count (not a literal 108), floored by the bytes that must come
  from HBM at the measured streaming rate of the SMs that take part, plus the measured
  overhead of the stream-K fix-up or the split-K sum where used;
* the prediction describes ONE launch that waits for its predecessor (what a caller's single
  call sees).  ``overlapped=True`` describes instead a chain of launches on distinct buffers
  flagged independent, which share the machine: a property of how the caller launches, passed
  in by the caller (the timing harness does so for shapes it rotates buffers for).

The dictionary is one Python literal (``str(dict)``), written where the reference writes it:
``build/prof_dict/<backend>_cost_model.dict``.
"""
import math

TILE_M = 128
TILE_K = 64
GEMM_TILE_NS = (256, 128, 64, 32, 16)
GEMV_VARIANTS = ((2, 4), (1, 4), (1, 8), (2, 2))   # (rows per warp, 16-byte loads in flight per row)
GEMV_SPLITS = (1, 2, 4, 8)
DEFAULT_SMS = 148
ROTATE_INTENSITY = 300.0    # flop per operand byte up to which the harness rotates operand sets and overlaps launches
SPLIT_MODES = (2, 3, 4)     # mode values that mean split-K over that many slices

# FP32 SIMT tiles: (BM, BN, BK, TM, TN, stages), the analogue of the reference's
# (BM, BN, BK, TM, TN, WARP_ROW_THREAD, COPY_A, COPY_B) keys (build_Ampere_FP32.py:37-63)
SGEMM_TILES = ((128, 128, 16, 8, 8, 4), (128, 128, 32, 8, 8, 3), (128, 64, 16, 8, 4, 4), (128, 64, 32, 8, 4, 3),
               (64, 128, 16, 4, 8, 4),
               (128, 128, 16, 8, 8, 2), (128, 64, 16, 8, 4, 2), (64, 128, 16, 4, 8, 2), (64, 64, 16, 4, 4, 2),
               (32, 64, 16, 4, 4, 2))


def is_valid_config(tile_n, swap_ab, mode, stages):
    """Analogue of is_valid_config (build_Ampere_FP16.py:30-39): what the library can launch."""
    return ((tile_n in GEMM_TILE_NS or tile_n in PAIR_TILE_NS) and swap_ab in (0, 1) and
            (mode in (0, 1) or mode in SPLIT_MODES) and 0 <= stages <= 8)


def max_stages(tile_n):
    budget = 227 * 1024 - 1024 - 256 - 32768     # alignment slack, barriers, output staging
    return min(8, budget // (TILE_M * TILE_K * 2 + tile_n * TILE_K * 2))


def pair_max_stages(tile_n):
    budget = 227 * 1024 - 1024 - 256 - 32768
    return min(8, budget // (TILE_M * TILE_K * 2 + (tile_n // 2) * TILE_K * 2))


# two CTAs share a 256 x 256 tile (tcgen05.mma.cta_group::2); each CTA holds 128 rows.
# The 256 x 192 pair tile exists for tile counts that quantise badly at 256 x 256.
PAIR_TILE_NS = (256, 192)
PAIR_KEYS = tuple((pair_max_stages(bn), TILE_M, bn, 2, 0, 0) for bn in PAIR_TILE_NS)
PAIR_KEY = PAIR_KEYS[0]


def gemm_keys():
    """Every GEMM configuration of the search space, as dictionary keys."""
    keys = []
    for bn in GEMM_TILE_NS:
        for swap in (0, 1):
            for mode in (0, 1):
                keys.append((max_stages(bn), TILE_M, bn, 1, swap, mode))
    for bn in (256, 128, 64):
        for split in SPLIT_MODES:
            keys.append((max_stages(bn), TILE_M, bn, 1, 0, split))
    keys.extend(PAIR_KEYS)
    return keys


def gemv_keys():
    return [(0, 1, rpw, unroll, 0, split) for (rpw, unroll) in GEMV_VARIANTS for split in GEMV_SPLITS]


def sgemm_keys():
    """(BM, BN, BK, TM, TN, stages, 0, 0): stages 2 = register-staged double buffer, >= 3 = cp.async ring."""
    return [(bm, bn, bk, tm, tn, st, 0, 0) for (bm, bn, bk, tm, tn, st) in SGEMM_TILES]


# ----------------------------------------------------------------------------- prediction
def _param(prof_dict, name, default):
    return prof_dict.get((name,), default)


def _lone_skinny_time(prof_dict, bn, stages, split, M, N, K, batch, sms):
    """One row block of A against a long weight matrix, launched alone: bound by the bytes the CTAs keep in
    flight (a CTA holds `stages` slabs; HBM answers a slab about 1.8 us after the request under load) or by the
    HBM rate, plus launch and drain (6 us) and the split-K sum."""
    tiles = -(-N // bn) * batch
    if split > 1 and (tiles * split > sms or -(-K // TILE_K) // split < 8):
        return float("inf")
    a_bytes, b_bytes = 2.0 * batch * M * K, 2.0 * batch * N * K
    slab_bytes = (min(M, TILE_M) + bn) * TILE_K * 2.0
    cta_rate = min(180e9, stages * slab_bytes / _param(prof_dict, "hbm_latency_s", 1.8e-6))
    ctas = min(tiles * split, sms)
    rounds = -(-tiles * split // sms)
    in_flight = (b_bytes + a_bytes * -(-N // bn)) / (ctas * cta_rate) * rounds
    t = max(in_flight, (a_bytes + b_bytes) / (_param(prof_dict, "hbm_lone_gbs", 5500.0) * 1e9)) + \
        _param(prof_dict, "lone_fixed", 6e-6)
    if split > 1:
        a, b = prof_dict.get(("splitk_overhead", bn), (2e-6 + 4e-6 * bn / 256.0, 1.5e-6 * bn / 256.0))
        live = min(4, (min(M, TILE_M) + 31) // 32) / 4.0
        t += 2e-6 + max(a - 2e-6 + b * split, 0.0) * live
    return t


def gemm_time(prof_dict, key, M, N, K, batch=1, conv=False, overlapped=False, operand_bytes=None):
    """Predicted seconds of one GEMM launch with configuration `key` (inf if inapplicable).  `operand_bytes`: what the
    launch really moves when that is not 2 (MK + NK + MN) -- an implicit-GEMM convolution reads every input pixel once,
    not once per filter tap."""
    stages, tm, bn, group, swap, mode = key
    split = mode if mode in SPLIT_MODES else 1
    if split > 1:
        if group != 1 or swap:
            return float("inf")
        mode = 0
    val = prof_dict.get((stages, tm, bn, group, swap, mode)) or prof_dict.get((stages, tm, bn, group, 0, 0))
    if val is None:
        return float("inf")
    t_fixed, t_slab = val
    if conv:
        # conv = True: any geometry (gathering producer possible): plain tiles only.  conv = "im2col": the
        # activations arrive through the im2col tensor map, which also serves the swapped tile (output channels
        # on the 128 rows, bn pixels per box) and split-K.
        # (64 or fewer output channels would fill half of the swapped tile's 128 rows and still pay its epilogue:
        # measured 23.1 us against 20.7 on 3 x 3, 64 -> 64 channels, 56 x 56)
        if swap and (conv != "im2col" or bn < 64 or N <= 64 or ("conv_slab_swap", bn) not in prof_dict):
            return float("inf")
        if split > 1 and conv != "im2col":
            return float("inf")
        t_slab = max(t_slab, prof_dict.get(("conv_slab_swap" if swap else "conv_slab", bn), t_slab))
        t_fixed = max(t_fixed, prof_dict.get(("conv_fixed_swap" if swap else "conv_fixed", bn), t_fixed))
    sms = _param(prof_dict, "sm_count", DEFAULT_SMS)
    pm, pn = (N, M) if swap else (M, N)
    # the library's own rules, which the slab figures cannot express: a tile twice as wide as the problem does the
    # narrower tile's work at a wider tile's price, and swapping operands only pays when the row count is the skinny
    # dimension (a convolution's swapped tile is covered above)
    if bn > 16 and bn // 2 >= pn:
        return float("inf")
    if swap and not conv and M > 64:
        return float("inf")
    if group == 2:
        if conv or swap or mode or pm <= tm or K < 8 * TILE_K:   # short K is epilogue bound: pairs gain nothing
            return float("inf")
        tm, sms = 2 * tm, sms // 2      # a pair of SMs is one scheduling slot for a 256-row tile
    tiles_m, tiles_n = -(-pm // tm), -(-pn // bn)
    tiles = tiles_m * tiles_n * batch
    nkb = -(-K // TILE_K)
    if not conv and group == 1 and not swap and mode == 0 and M <= tm and N >= 1024 and nkb >= 8 and \
            (split > 1 or not overlapped):
        return _lone_skinny_time(prof_dict, bn, stages, split, M, N, K, batch, sms)
    if not conv and group == 1 and not swap and mode == 0 and M <= tm and ("skinny_fixed",) in prof_dict:
        # overlapped launches of one row block of A against a long weight matrix: B streams from HBM once,
        # the A box only carries M rows; bounded by the HBM rate reached with wide boxes or by what one CTA takes in
        if bn < 128 and N >= 1024:
            return float("inf")     # narrow boxes stream B at a fraction of the rate (measured 30 us vs 20 at bn 64)
        bytes_ = 2.0 * batch * (M * K + N * K + M * N)
        slab_bytes = (min(M, tm) + bn) * TILE_K * 2.0
        # the HBM rate grows a little with the number of streaming CTAs (measured 4.6 TB/s with 16..43, 5.6 with 148)
        wide = _param(prof_dict, "hbm_wide_gbs", 5300.0)
        if bn < 256:     # narrower boxes: their own measured rate where the profile has it
            wide = prof_dict.get(("hbm_wide_gbs", bn), 0.85 * wide)
        hbm = wide * 1e9 * (0.8 + 0.2 * min(tiles, sms) / sms)
        t_hbm = bytes_ / hbm
        t_cta = -(-tiles // sms) * nkb * slab_bytes / (_param(prof_dict, "wide_gbs_per_sm", 400.0) * 1e9)
        # every CTA pulls the same A rows: those lines are a hot spot in L2, which then delivers
        # only about half of what it gives a square GEMM
        t_l2 = tiles * nkb * slab_bytes / (_param(prof_dict, "skinny_l2_gbs", 9300.0) * 1e9)
        return prof_dict[("skinny_fixed",)] + max(t_hbm, t_cta, t_l2)
    rounds, tail = divmod(tiles, sms)
    if split > 1:
        # K cut into `split` slices, one work item each, all resident at once; the last arriver sums
        if tiles * split > sms or nkb // split < 4:
            return float("inf")
        slabs = -(-nkb // split)
        active = tiles * split
        a, b = prof_dict.get(("splitk_overhead", bn), (2e-6 + 4e-6 * bn / 256.0, 1.5e-6 * bn / 256.0))
        extra = a + b * split
    elif mode == 0:
        slabs = (rounds + (1 if tail else 0)) * nkb
        active = min(tiles, sms)
        extra = 0.0
    else:
        if tail == 0 or nkb < 2:
            return float("inf")      # identical to mode 0: keep one entry
        slabs = rounds * nkb + max(-(-tail * nkb // sms), min(4, nkb))
        active = min(tiles * nkb, sms)
        extra = prof_dict.get(("streamk_overhead", bn), 8e-6)
    if group == 2:
        active *= 2
    t = t_fixed + slabs * t_slab + extra
    bytes_ = operand_bytes if operand_bytes is not None else 2.0 * batch * (M * K + N * K + M * N)
    if (overlapped and not conv and mode == 0 and split == 1 and not swap and min(M, N) > TILE_M and tiles < sms
            and 2.0 * batch * M * N * K / bytes_ <= ROTATE_INTENSITY):
        # A chain of independent launches over distinct operand sets: a launch that leaves SMs free and
        # needs no workspace overlaps its neighbours, so the chain advances by the launch's share of the
        # machine, not by its latency, and the floor is the HBM rate this kernel reaches with every SM
        # streaming (below the GEMV's).  Launches with a workspace are ordered on the stream and keep their
        # full latency.  Not applied to swapped operands: those stream a long matrix through few CTAs and
        # are bound by what one CTA takes in, which overlap does not change.
        return max(t * max(tiles / sms, 1.0 / 16.0), bytes_ / (_param(prof_dict, "hbm_wide_gbs", 5300.0) * 1e9))
    # HBM floor: operand bytes at the streaming rate of the SMs that take part
    per_sm = _param(prof_dict, "dram_gbs_per_sm", 40.0) * 1e9
    hbm = _param(prof_dict, "hbm_gbs", 6000.0) * 1e9
    t_mem = t_fixed + bytes_ / min(hbm, active * per_sm)
    return max(t, t_mem)


def gemv_time(prof_dict, key, rows, K, m):
    val = prof_dict.get(key)
    if val is None or m > 8:
        return float("inf")
    t_fixed, s_per_byte = val
    split = key[5]
    if split > 1 and K // split < 256:
        return float("inf")
    bytes_ = 2.0 * (rows * K + m * K + m * rows)
    # m right-hand sides multiply the arithmetic per streamed byte and the SIMT kernel becomes issue bound:
    # measured on 4096 x 1024 weights, the streaming part takes 1.33x (m = 2), 2.0x (4), 3.6x (6), 4.4x (8)
    # of its m = 1 time
    growth = 1.0 + 0.35 * (m - 1) if m <= 4 else 0.6 * m
    return t_fixed + bytes_ * s_per_byte * growth


def cost_model(prof_dict, M, N, K, batch=1, conv=False, overlapped=False, operand_bytes=None):
    """Best configuration key for C[M,N] = A[M,K] * B[N,K]^T; first element 0 means GEMV.

    Same call shape as the reference's cost_model(prof_dict, M, N, K)
    (Ampere_FP16_gemm.py:420-430), but K and the batch count enter the estimate.
    """
    best_key, best = None, float("inf")
    for key in prof_dict:
        if len(key) != 6:
            continue
        if key[0] == 0:
            if conv or batch != 1 or min(M, N) > 8:
                continue
            rows, m = (N, M) if M <= N else (M, N)
            t = gemv_time(prof_dict, key, rows, K, m)
        else:
            t = gemm_time(prof_dict, key, M, N, K, batch, conv, overlapped, operand_bytes)
        if t < best:
            best, best_key = t, key
    return best_key


def predicted_time(prof_dict, key, M, N, K, batch=1, conv=False, overlapped=False, operand_bytes=None):
    if key[0] == 0:
        rows, m = (N, M) if M <= N else (M, N)
        return gemv_time(prof_dict, key, rows, K, m)
    return gemm_time(prof_dict, key, M, N, K, batch, conv, overlapped, operand_bytes)


def sgemm_cost_model(prof_dict, M, N, K):
    """FP32: ceil(tiles / SMs) * K-slabs * profiled seconds per tile-slab (Ampere_FP32_gemm.py:89-99)."""
    sms = _param(prof_dict, "sm_count", DEFAULT_SMS)
    best_key, best = None, float("inf")
    for key, v in prof_dict.items():
        if len(key) != 8:
            continue
        bm, bn, bk = key[0], key[1], key[2]
        tiles = -(-M // bm) * -(-N // bn)
        t = math.ceil(tiles / sms) * -(-K // bk) * v
        if t < best:
            best, best_key = t, key
    return best_key


# ----------------------------------------------------------------------------- dictionary I/O
def save(prof_dict, path):
    import os
    os.makedirs(os.path.dirname(path), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        f.write(str(prof_dict))
    os.replace(tmp, path)          # a crash mid-profile never leaves a truncated dictionary


def load(path):
    with open(path) as f:
        return eval(f.readlines()[0])   # the reference's own loading idiom (benchmark_Ampere_FP16_gemm.py:10-12)
