"""In-process replacements for the reference's per-configuration executables.

The reference measures a configuration by spawning ``build/bin_fp16/gemm_<cfg> M N K`` and
reading token [-8] of its stdout (scripts/Ampere_FP16/profile_Ampere_FP16.py:36-39,
Ampere_FP16_gemm.py:438-441).  Here the same questions -- "how long does this configuration
take on this shape", "fill the dictionary", "run the predicted-best configuration" -- are
answered through the C ABI, with operands that are real seeded data and with rotating buffers
for memory-bound shapes so that they really come from HBM.
"""
import math
import os

import torch

from . import costmodel, ops
from ._lib import LAUNCH_INDEPENDENT, OP_CONV_F16, OP_GEMM_F16, OP_GEMM_F32, OP_GEMV_F16

ROTATE_BYTES = 300e6      # more than twice the 126 MB L2


def root_path():
    return os.getcwd()   # the reference resolves build/ against the working directory (build_Ampere_FP16.py:4)


def dict_path(backend):
    return os.path.join(root_path(), "build", "prof_dict", f"{backend}_cost_model.dict")


def require_gpu():
    if not torch.cuda.is_available():
        raise RuntimeError("the Helix B200 backends need a CUDA device; there is no CPU fallback")


def key_to_cfg(key, conv=False, prof_dict=None):
    """Dictionary key -> library configuration.  With the profiled dictionary at hand, the number of
    TMA-issuing warps is the one the profile found fastest for the tile width (("load_group", bn))."""
    if key[0] == 0:
        return ops.make_cfg(OP_GEMV_F16, tile_m=1, tile_n=key[2], tile_k=256, split_k=key[5], load_group=key[3])
    stages, tm, bn, group, swap, mode = key
    split = mode if mode in costmodel.SPLIT_MODES else 1
    lg = int((prof_dict or {}).get(("load_group", bn), 0)) if group == 1 else 0
    return ops.make_cfg(OP_CONV_F16 if conv else OP_GEMM_F16, tile_m=tm, tile_n=bn, tile_k=costmodel.TILE_K,
                        stages=0, cta_group=group, swap_ab=swap, stream_k=(1 if mode == 1 else 0), split_k=split,
                        load_group=lg)


def overlaps(M, N, K, batch=None):
    """True where time_gemm_f16 rotates operand sets and flags its launches independent, i.e. measures the
    throughput of overlapping launches rather than one launch's latency: the protocol flag the cost model
    takes from its caller."""
    b = batch or 1
    return 2.0 * b * M * N * K / (2.0 * b * (M * K + N * K + M * N)) <= costmodel.ROTATE_INTENSITY


def cost_model(prof_dict, M, N, K, batch=None, conv=False):
    """costmodel.cost_model for a shape that this harness is going to time (its protocol passed along)."""
    return costmodel.cost_model(prof_dict, M, N, K, batch or 1, conv, overlapped=overlaps(M, N, K, batch))


def predicted_time(prof_dict, key, M, N, K, batch=None, conv=False):
    return costmodel.predicted_time(prof_dict, key, M, N, K, batch or 1, conv, overlapped=overlaps(M, N, K, batch))


def _randn(shape, scale):
    return torch.randn(shape, device="cuda", dtype=torch.float16) * scale


def time_gemm_f16(M, N, K, cfg=None, batch=None, iters=20, lone=False):
    """Seconds per launch of the fp16 GEMM; operands rotate through > 2x L2 when the shape is memory-bound
    (launches on distinct buffer sets, flagged independent, overlap).  lone=True: one buffer set, every launch
    waiting for its predecessor -- what a caller's single call sees."""
    b = batch or 1
    bytes_ = 2.0 * b * (M * K + N * K + M * N)
    flops = 2.0 * b * M * N * K
    nbuf = 1 if (lone or flops / bytes_ > costmodel.ROTATE_INTENSITY) else int(ROTATE_BYTES // bytes_) + 1
    sa, sb, sc = ((M, K), (N, K), (M, N)) if batch is None else ((b, M, K), (b, N, K), (b, M, N))
    s = 1.0 / math.sqrt(K)
    bufs = [(_randn(sa, s), _randn(sb, s), torch.empty(sc, device="cuda", dtype=torch.float16)) for _ in range(nbuf)]
    ls = [ops.launch_gemm_f16(a, bb, c, cfg) for a, bb, c in bufs]
    if len(ls) > 1:
        for l in ls:
            l.flags = LAUNCH_INDEPENDENT     # rotating buffer sets: neighbours share nothing
    reps = max(1, 4 // len(ls))
    avg, _, _ = ops.time_launches(ls * reps, warmup=3, iters=iters, use_graph=True)
    return avg


def time_gemv_f16(rows, K, m, cfg=None, transposed=False, iters=30):
    bytes_ = 2.0 * (rows * K + m * K + m * rows)
    nbuf = int(ROTATE_BYTES // bytes_) + 1
    x = _randn((m, K), 1.0)
    ws = [_randn((rows, K), 0.02) for _ in range(nbuf)]
    oshape = (rows, m) if transposed else (m, rows)
    ys = [torch.empty(oshape, device="cuda", dtype=torch.float16) for _ in range(nbuf)]
    ls = [ops.launch_gemv_f16(w, x, y, cfg, out_transposed=transposed) for w, y in zip(ws, ys)]
    if len(ls) > 1:
        for l in ls:
            l.flags = LAUNCH_INDEPENDENT
    reps = max(1, 4 // len(ls))
    avg, _, _ = ops.time_launches(ls * reps, warmup=3, iters=iters, use_graph=True)
    return avg


def time_conv_f16(batch, IC, H, W, OC, kH, kW, stride, pad, cfg=None, iters=20):
    C = ops.conv_stored_channels(IC, H, W, OC, kH, kW, stride, pad)    # zero channels pad the pixel to 8 or 16 bytes
    x = torch.rand((batch, H, W, C), device="cuda", dtype=torch.float16) * 2 - 1
    w = _randn((OC, kH, kW, C), math.sqrt(2.0 / (IC * kH * kW)))
    if C != IC:
        x[..., IC:] = 0
        w[..., IC:] = 0
    Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
    y = torch.empty((batch, Ho, Wo, OC), device="cuda", dtype=torch.float16)
    l = ops.launch_conv2d_f16(x, w, y, stride, pad, cfg)
    avg, _, _ = ops.time_launches([l] * 4, warmup=3, iters=iters, use_graph=True)
    return avg


def time_gemv_f32(rows, K, m, cfg=None, transposed=False, iters=30):
    """Seconds per launch of the fp32 GEMV with W rotating through > 2x L2."""
    bytes_ = 4.0 * (rows * K + m * K + m * rows)
    nbuf = int(ROTATE_BYTES // bytes_) + 1
    x = torch.rand((m, K), device="cuda") * 2 - 1
    ws = [torch.rand((rows, K), device="cuda") * 2 - 1 for _ in range(nbuf)]
    oshape = (rows, m) if transposed else (m, rows)
    ys = [torch.empty(oshape, device="cuda") for _ in range(nbuf)]
    ls = [ops.launch_gemv_f32(w, x, y, cfg, out_transposed=transposed) for w, y in zip(ws, ys)]
    reps = max(1, 4 // len(ls))
    avg, _, _ = ops.time_launches(ls * reps, warmup=3, iters=iters, use_graph=True)
    return avg


def time_gemm_f32(M, N, K, cfg=None, iters=10):
    a = torch.rand((M, K), device="cuda") * 2 - 1
    b = torch.rand((K, N), device="cuda") * 2 - 1
    c = torch.empty((M, N), device="cuda")
    avg, _, _ = ops.time_launches([ops.launch_gemm_f32(a, b, c, False, cfg)] * 2, warmup=2, iters=iters, use_graph=True)
    return avg


# ----------------------------------------------------------------------------- profiling
def _two_point(t1, s1, t2, s2):
    slab = max((t2 - t1) / (s2 - s1), 1e-9)
    return max(t1 - s1 * slab, 0.0), slab


def profile_fp16(fast=False, progress=None):
    """Fill the fp16 dictionary.  fast=True is the 'changed_profile' mode: probe the widest and the
    64-wide tile only and interpolate the rest (the reference's fast mode extrapolates
    BLOCK > WARP tiles from BLOCK == WARP ones, changed_profile_Ampere_FP16.py:27-54)."""
    require_gpu()
    sms = ops.device_info().sm_count
    d = {("sm_count",): sms}
    tick = progress or (lambda: None)

    def cfg(bn, swap=0, mode=0):
        return ops.make_cfg(OP_GEMM_F16, 128, bn, 64, swap_ab=swap, stream_k=mode, load_group=0)

    measured = {}
    wide = (256, 64) if fast else (256, 128, 64)
    for bn in wide:                                  # L2-friendly square problem, two K values
        M = N = 4096
        tiles = (M // 128) * (N // bn)
        waves = -(-tiles // sms)
        t1 = time_gemm_f16(M, N, 512, cfg(bn)); tick()
        t2 = time_gemm_f16(M, N, 4096, cfg(bn)); tick()
        measured[bn] = _two_point(t1, waves * 8, t2, waves * 64)
    if fast:                                         # interpolate 128 between 64 and 256
        f64, f256 = measured[64], measured[256]
        measured[128] = tuple(a + (b - a) * (128 - 64) / (256 - 64) for a, b in zip(f64, f256))
    # CTA pairs on 256 x BN tiles: 16 x ceil(4096 / BN) pair tiles on sms/2 pairs
    for pkey in costmodel.PAIR_KEYS:
        bn = pkey[2]
        pair_cfg = ops.make_cfg(OP_GEMM_F16, 128, bn, 64, cta_group=2)
        pair_waves = -(-(16 * -(-4096 // bn)) // (sms // 2))
        t1 = time_gemm_f16(4096, 4096, 512, pair_cfg); tick()
        t2 = time_gemm_f16(4096, 4096, 4096, pair_cfg); tick()
        d[pkey] = tuple(float(v) for v in _two_point(t1, pair_waves * 8, t2, pair_waves * 64))
    # one row block of A against a long B with the widest tile: what a single CTA takes in (16 CTAs,
    # two K values) and the HBM rate with every SM streaming
    t1 = time_gemm_f16(8, 4096, 2048, cfg(256)); tick()
    t2 = time_gemm_f16(8, 4096, 8192, cfg(256)); tick()
    slab_bytes = (8 + 256) * 64 * 2.0
    d[("wide_gbs_per_sm",)] = float((8192 - 2048) / 64 * slab_bytes / max(t2 - t1, 1e-9) / 1e9)
    per_byte = max(t2 - t1, 1e-9) / (2.0 * 4096 * (8192 - 2048))
    d[("skinny_fixed",)] = float(max(t1 - 2.0 * 4096 * 2048 * per_byte, 2.5e-6))
    t = time_gemm_f16(128, 8192, 4096, cfg(64)); tick()      # 128 CTAs, all reading the same 128 rows of A
    d[("skinny_l2_gbs",)] = float(128 * 64 * (128 + 64) * 64 * 2.0 / max(t - d[("skinny_fixed",)], 1e-9) / 1e9)
    t = time_gemm_f16(16, 256 * sms, 4096, cfg(256)); tick()
    d[("hbm_wide_gbs",)] = float(2.0 * (16 * 4096 + 256 * sms * 4096 + 16 * 256 * sms) /
                                  max(t - d[("skinny_fixed",)], 1e-9) / 1e9)
    # the same stream through 128-row boxes (twice the tensor copies per byte): measurably slower
    t = time_gemm_f16(16, 256 * sms, 4096, cfg(128)); tick()
    d[("hbm_wide_gbs", 128)] = float(2.0 * (16 * 4096 + 256 * sms * 4096 + 16 * 256 * sms) /
                                      max(t - d[("skinny_fixed",)], 1e-9) / 1e9)
    skinny = {}
    for bn in ((16,) if fast else (32, 16)):          # skinny M on the UMMA N axis: everything streams from DRAM
        N = 128 * sms
        t1 = time_gemm_f16(bn, N, 1024, cfg(bn, swap=1)); tick()
        t2 = time_gemm_f16(bn, N, 8192, cfg(bn, swap=1)); tick()
        skinny[bn] = _two_point(t1, 16, t2, 128)
    if fast:
        skinny[32] = skinny[16]
    # per-SM DRAM streaming rate from the narrowest tile: each CTA pulls 128 rows x 64 halves per slab
    d[("dram_gbs_per_sm",)] = (128 * 64 * 2 + 16 * 64 * 2) / skinny[16][1] / 1e9
    for bn in costmodel.GEMM_TILE_NS:
        val = measured.get(bn) or skinny.get(bn)
        for swap in (0, 1):
            for mode in (0, 1):
                d[(costmodel.max_stages(bn), 128, bn, 1, swap, mode)] = tuple(float(v) for v in val)
        if bn >= 64:
            for split in costmodel.SPLIT_MODES:      # same slab figures; the sum's cost is ("splitk_overhead", bn)
                d[(costmodel.max_stages(bn), 128, bn, 1, 0, split)] = tuple(float(v) for v in val)
    # stream-K: measured excess over the slab model on a half-wave problem
    for bn in wide:
        M, N, K = 128 * (sms // 2), bn, 4096
        t = time_gemm_f16(M, N, K, cfg(bn, mode=1)); tick()
        tf, ts = measured[bn]
        d[("streamk_overhead", bn)] = max(t - (tf + 32 * ts), 2e-6)
    if fast:
        d[("streamk_overhead", 128)] = 0.5 * (d[("streamk_overhead", 64)] + d[("streamk_overhead", 256)])
    # convolution: slope per slab of the gathering producer (3x3, 28x28, batch 32: 196 tiles)
    for bn in wide:
        ccfg = ops.make_cfg(OP_CONV_F16, 128, bn, 64)
        waves = -(-196 * max(1, 1) // sms)
        t1 = time_conv_f16(32, 64, 28, 28, bn, 3, 3, 1, 1, ccfg); tick()
        t2 = time_conv_f16(32, 256, 28, 28, bn, 3, 3, 1, 1, ccfg); tick()
        fx, sl = _two_point(t1, waves * 9, t2, waves * 36)
        d[("conv_slab", bn)] = sl
        d[("conv_fixed", bn)] = float(fx)      # launch, im2col set-up and epilogue of a convolution launch
    if fast:
        d[("conv_slab", 128)] = 0.5 * (d[("conv_slab", 64)] + d[("conv_slab", 256)])
        d[("conv_fixed", 128)] = 0.5 * (d[("conv_fixed", 64)] + d[("conv_fixed", 256)])
    # swapped convolution tiles (output channels on the 128 rows, bn pixels per im2col box): slope per slab on
    # 128 output channels, 28 x 28, batch 32 (25088 pixels)
    for bn in ((256,) if fast else (256, 128)):
        ccfg = ops.make_cfg(OP_CONV_F16, 128, bn, 64, swap_ab=1)
        waves = -(-(-(-25088 // bn)) // sms)
        t1 = time_conv_f16(32, 64, 28, 28, 128, 3, 3, 1, 1, ccfg); tick()
        t2 = time_conv_f16(32, 256, 28, 28, 128, 3, 3, 1, 1, ccfg); tick()
        fx, sl = _two_point(t1, waves * 9, t2, waves * 36)
        d[("conv_slab_swap", bn)] = sl
        d[("conv_fixed_swap", bn)] = float(fx)
    # split-K: what the slot round trip and the last arriver's sum add, from two slice counts on a quarter-wave
    # problem: t - (fixed + slabs * slab) = a + b * S
    for bn in wide:
        M, N, K = 128 * (sms // 4), bn, 4096
        tf, ts = measured[bn]
        over = {}
        for S in (2, 4):
            c = ops.make_cfg(OP_GEMM_F16, 128, bn, 64, split_k=S)
            over[S] = time_gemm_f16(M, N, K, c) - (tf + (64 // S) * ts); tick()
        b = max((over[4] - over[2]) / 2.0, 0.0)
        d[("splitk_overhead", bn)] = (float(max(over[2] - 2.0 * b, 1e-6)), float(b))
    if fast:
        d[("splitk_overhead", 128)] = tuple(0.5 * (x + y) for x, y in zip(d[("splitk_overhead", 64)], d[("splitk_overhead", 256)]))
    # search over the fields the key does not carry: TMA-issuing warps per CTA (load_group 1..3) on a tensor-bound
    # probe, kept per tile width and applied by key_to_cfg; ring depth on the same probe (recorded: the deepest ring
    # that fits is never slower, which is why the key space holds one depth per width)
    if not fast:
        for bn in wide:
            best = None
            for lg in (1, 2, 3):
                t = time_gemm_f16(4096, 4096, 1024, ops.make_cfg(OP_GEMM_F16, 128, bn, 64, load_group=lg)); tick()
                d[("load_group_probe", bn, lg)] = float(t)
                if best is None or t < best[1] * 0.99:
                    best = (lg, t)
            d[("load_group", bn)] = best[0]
            smax = costmodel.max_stages(bn)
            for st in sorted({2, max(2, smax // 2), smax}):
                t = time_gemm_f16(4096, 4096, 1024, ops.make_cfg(OP_GEMM_F16, 128, bn, 64, stages=st)); tick()
                d[("stages_probe", bn, st)] = float(t)
    # GEMV: fixed cost and seconds per streamed byte for each variant
    variants = costmodel.GEMV_VARIANTS[:1] if fast else costmodel.GEMV_VARIANTS
    best_rate = 0.0
    for (rpw, unroll) in variants:
        for split in costmodel.GEMV_SPLITS:
            c = ops.make_cfg(OP_GEMV_F16, tile_m=1, tile_n=rpw, tile_k=256, split_k=split, load_group=unroll)
            t1 = time_gemv_f16(2048, 4096, 1, c); tick()
            t2 = time_gemv_f16(16384, 8192, 1, c); tick()
            b1, b2 = 2.0 * (2048 * 4096), 2.0 * (16384 * 8192)
            per_byte = max((t2 - t1) / (b2 - b1), 1e-15)
            fixed = max(t1 - b1 * per_byte, 0.0)
            d[(0, 1, rpw, unroll, 0, split)] = (float(fixed), float(per_byte))
            best_rate = max(best_rate, b2 / t2 / 1e9)
    d[("hbm_gbs",)] = best_rate
    return d


def sgemm_key_to_cfg(key):
    """(BM, BN, BK, TM, TN, stages, 0, 0) -> library configuration (stages 0 reads as the 2-buffer kernel)."""
    bm, bn, bk, tm, tn = key[:5]
    return ops.make_cfg(OP_GEMM_F32, tile_m=bm, tile_n=bn, tile_k=bk, thread_m=tm, thread_n=tn,
                        stages=(key[5] if len(key) > 5 and key[5] else 2))


def profile_fp32(fast=False, progress=None):
    require_gpu()
    sms = ops.device_info().sm_count
    d = {("sm_count",): sms}
    size = 1024 if fast else 2048
    for key in costmodel.sgemm_keys():
        bm, bn, bk = key[:3]
        c = sgemm_key_to_cfg(key)
        try:
            t = time_gemm_f32(size, size, size, c)
            tiles = -(-size // bm) * -(-size // bn)
            d[key] = float(t / (math.ceil(tiles / sms) * (size // bk)))
        except Exception:
            d[key] = float("inf")   # a configuration that fails to run never wins (profile_Ampere_FP32.py:41-45)
        if progress:
            progress()
    return d


# ----------------------------------------------------------------------------- "run the winner"
def gemm_f16_result(prof_dict, M, N, K, batch=None):
    """(cost_ms, tflops) of the predicted-best configuration, the contract of
    get_Ampere_FP16_gemm_Helix_result (Ampere_FP16_gemm.py:432-441, cuda branch: milliseconds)."""
    require_gpu()
    key = cost_model(prof_dict, M, N, K, batch)
    if key is None:
        raise RuntimeError("empty cost-model dictionary: run profile_template.py first")
    if key[0] == 0:
        rows, m, transposed = (N, M, False) if M <= N else (M, N, True)
        Kp = (K + 7) // 8 * 8
        t = time_gemv_f16(rows, Kp, m, key_to_cfg(key), transposed)
    else:
        Kp = (K + 7) // 8 * 8      # leading dimensions follow the 16-byte rule; the padding columns are zero work
        t = time_gemm_f16(M, N, Kp, key_to_cfg(key, prof_dict=prof_dict), batch)
    cost_ms = t * 1e3
    return cost_ms, 2.0 * M * N * K * (batch or 1) / 1e9 / cost_ms


def time_key_f16(key, M, N, K):
    """Seconds of one fp16 GEMM under the dictionary key `key` (a GEMV key runs the GEMV kernel; it needs
    min(M, N) <= 8).  What the reference's ablation scripts do by spawning one executable per candidate
    (scripts/Ampere_FP16/candidate_performance_curve.py:22-31)."""
    require_gpu()
    Kp = (K + 7) // 8 * 8
    if key[0] == 0:
        rows, m, transposed = (N, M, False) if M <= N else (M, N, True)
        if m > 8:
            raise ValueError("the GEMV kernel takes at most 8 right-hand sides")
        return time_gemv_f16(rows, Kp, m, key_to_cfg(key), transposed)
    return time_gemm_f16(M, N, Kp, key_to_cfg(key))


def gemv_passes_time(M, N, K, cfg=None):
    """Seconds of y[M,N] = x[M,K] W[N,K]^T done by the GEMV kernel alone: ceil(M/8) launches of at most 8
    right-hand sides each, timed as one chain (the reference's gemv executable loops over M itself,
    scripts/Ampere_FP16/TensorCore_CUDACore_Adaptive.py:48-54).  Pass a GEMV `cfg` to keep the library
    from serving 3..8 right-hand sides with the tensor-core kernel."""
    require_gpu()
    Kp = (K + 7) // 8 * 8
    nbuf = int(ROTATE_BYTES // (2.0 * N * Kp)) + 1
    x = _randn((M, Kp), 1.0)
    chains = []
    for _ in range(nbuf):
        w = _randn((N, Kp), 0.02)
        y = torch.empty((M, N), device="cuda", dtype=torch.float16)
        for m0 in range(0, M, 8):
            m1 = min(M, m0 + 8)
            l = ops.launch_gemv_f16(w, x[m0:m1], y[m0:m1], cfg)
            l.flags = LAUNCH_INDEPENDENT          # passes write disjoint rows of y and only read W and x
            chains.append(l)
    avg, _, _ = ops.time_launches(chains, warmup=3, iters=20, use_graph=True)
    return avg * (-(-M // 8))


def conv_f16_result(prof_dict, batch, IC, H, W, OC, kH, kW, stride, pad):
    """(cost_ms, tflops) of one NHWC convolution as a single implicit GEMM
    (get_Ampere_FP16_conv_Helix_result, Ampere_FP16_conv.py:431-446: im2col time + GEMM time)."""
    require_gpu()
    Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
    M, N, K = batch * Ho * Wo, OC, IC * kH * kW
    as_gemm = kH == 1 and kW == 1 and stride == 1 and pad == 0
    C = ops.conv_stored_channels(IC, H, W, OC, kH, kW, stride, pad)
    if ops.conv_has_fixed_kernel(batch, C, H, W, OC, kH, kW, stride, pad):   # nothing for the cost model to pick
        cost_ms = time_conv_f16(batch, IC, H, W, OC, kH, kW, stride, pad) * 1e3
        return cost_ms, 2.0 * M * N * K / 1e9 / cost_ms
    im2col = C % 64 == 0 and batch * H * W * C * 2 >= 131072 and stride <= 8      # the library's tensor-map rule
    # the convolution harness times one buffer set with ordered launches: a lone launch
    real_bytes = 2.0 * (batch * H * W * C + OC * kH * kW * C + M * N)        # x, w and y once each
    key = costmodel.cost_model(prof_dict, M, N, (K + 7) // 8 * 8, 1,
                               conv=False if as_gemm else ("im2col" if im2col else True), operand_bytes=real_bytes)
    if key is None or key[0] == 0:
        key = (costmodel.max_stages(128), 128, 128, 1, 0, 0)
    t = time_conv_f16(batch, IC, H, W, OC, kH, kW, stride, pad, key_to_cfg(key, conv=True, prof_dict=prof_dict))
    cost_ms = t * 1e3
    return cost_ms, 2.0 * M * N * K / 1e9 / cost_ms


def gemm_f32_result(prof_dict, M, N, K):
    require_gpu()
    if min(M, N) <= 8 and max(M, N) >= 64:
        # up to eight rows or columns: the weight matrix is streamed once by the fp32 GEMV (the reference keeps
        # a GEMV template for this case, src_template/Ampere_FP32/gemv_template_fp32.cu, but never builds it)
        Kp = (K + 3) // 4 * 4
        rows, m, transposed = (N, M, False) if M <= N else (M, N, True)
        t = time_gemv_f32(rows, Kp, m, None, transposed)
        return t * 1e3, 2.0 * M * N * K / 1e9 / (t * 1e3)
    key = costmodel.sgemm_cost_model(prof_dict, M, N, K)
    if key is None:
        raise RuntimeError("empty cost-model dictionary: run profile_template.py -b Ampere_FP32 first")
    t = time_gemm_f32(M, N, K, sgemm_key_to_cfg(key))
    cost_ms = t * 1e3
    return cost_ms, 2.0 * M * N * K / 1e9 / cost_ms


def time_conv_f32(batch, IC, H, W, OC, kH, kW, stride, pad, cfg=None, iters=10):
    """Seconds of one true-fp32 NHWC convolution: weight transpose + column matrix + FFMA GEMM."""
    x = torch.rand((batch, H, W, IC), device="cuda") * 2 - 1
    w = torch.randn((OC, kH, kW, IC), device="cuda") * math.sqrt(2.0 / (IC * kH * kW))
    Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
    y = torch.empty((batch, Ho, Wo, OC), device="cuda")
    l = ops.launch_conv2d_f32(x, w, y, stride, pad, cfg)
    avg, _, _ = ops.time_launches([l] * 2, warmup=2, iters=iters, use_graph=True)
    return avg


def conv_f32_result(prof_dict, batch, IC, H, W, OC, kH, kW, stride, pad):
    """(cost_ms, tflops) of one fp32 convolution the reference's way: explicit column matrix, then the GEMM on
    M = B*Ho*Wo, N = OC, K = IC*kH*kW with the configuration the cost model picks for that shape
    (Ampere_FP32_conv.py:101-113); the time covers all three kernels."""
    require_gpu()
    Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
    M, N, K = batch * Ho * Wo, OC, IC * kH * kW
    key = costmodel.sgemm_cost_model(prof_dict, M, N, K)
    if key is None:
        raise RuntimeError("empty cost-model dictionary: run profile_template.py -b Ampere_FP32 first")
    t = time_conv_f32(batch, IC, H, W, OC, kH, kW, stride, pad, sgemm_key_to_cfg(key))
    cost_ms = t * 1e3
    return cost_ms, 2.0 * M * N * K / 1e9 / cost_ms


# ----------------------------------------------------------------------------- sharded-sweep workers
def _bind(device):
    require_gpu()
    torch.cuda.set_device(int(device))


def worker_gemm_f16(device, unit, prof_dict):
    _bind(device)
    M, N, K = unit[:3]
    cost, tflops = gemm_f16_result(prof_dict, M, N, K, unit[3] if len(unit) > 3 else None)
    return {"shape": list(unit), "ms": cost, "tflops": tflops}


def worker_conv_f16(device, unit, prof_dict):
    _bind(device)
    cost, tflops = conv_f16_result(prof_dict, *unit)
    return {"shape": list(unit), "ms": cost, "tflops": tflops}


def worker_gemm_f32(device, unit, prof_dict):
    _bind(device)
    cost, tflops = gemm_f32_result(prof_dict, *unit[:3])
    return {"shape": list(unit), "ms": cost, "tflops": tflops}


def worker_conv_f32(device, unit, prof_dict):
    _bind(device)
    cost, tflops = conv_f32_result(prof_dict, *unit)
    return {"shape": list(unit), "ms": cost, "tflops": tflops}


def run_shape_list(units, worker, prof_dict, gpus=1, predicted=None, journal=None):
    """Rows (ordered like `units`) of a sweep over 1..N GPUs of this box.  With `journal` (a JSONL path) every
    finished shape is appended as one line and shapes already present there are not run again, so a sweep
    that was interrupted resumes where it stopped."""
    from . import shard
    if gpus <= 1:
        import json
        done = shard.read_journal(journal)
        rows = []
        for i, u in enumerate(units):
            if i in done and list(done[i].get("shape", [])) == list(u):
                rows.append(done[i])
                continue
            row = dict(worker(torch.cuda.current_device() if torch.cuda.is_available() else 0, u, prof_dict))
            row["index"] = i
            if journal:
                with open(journal, "a") as f:
                    f.write(json.dumps(row) + "\n")
            rows.append(row)
        return rows
    rows, stats = shard.run_sharded(units, worker, list(range(gpus)), costs=predicted, journal=journal,
                                    fn_args=(prof_dict,))
    if stats["unfinished"]:
        raise RuntimeError(f"sweep incomplete: {stats}")
    return [rows[i] for i in range(len(units))]


# ----------------------------------------------------------------------------- vendor comparators (context only)
def time_torch(fn, iters=20):
    """Seconds per call of a torch operation: `iters` calls captured in a CUDA graph and replayed (so that a
    vendor kernel of a few microseconds is not rated by the host's launch rate); eager calls if capture fails."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    graph = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        graph = g
    except Exception:
        graph = None
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph is not None:
        graph.replay()
        torch.cuda.synchronize()
        reps = 3
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / (iters * reps)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / iters


def cublas_gemm_result(M, N, K, dtype=torch.float16):
    """cuBLAS through torch.matmul: the comparator row of the reference's cublas_f16.cu / cublas_f32.cu."""
    require_gpu()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        a = torch.randn((M, K), device="cuda", dtype=dtype)
        b = torch.randn((N, K), device="cuda", dtype=dtype)
        t = time_torch(lambda: torch.matmul(a, b.t()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    cost_ms = t * 1e3
    return cost_ms, 2.0 * M * N * K / 1e9 / cost_ms


def cudnn_conv_result(batch, IC, H, W, OC, kH, kW, stride, pad, dtype=torch.float16):
    """cuDNN through torch conv2d in channels-last: the comparator row of cudnn_fp16.cu / cudnn_fp32.cu."""
    require_gpu()
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        x = torch.randn((batch, IC, H, W), device="cuda", dtype=dtype).contiguous(memory_format=torch.channels_last)
        w = torch.randn((OC, IC, kH, kW), device="cuda", dtype=dtype).contiguous(memory_format=torch.channels_last)
        t = time_torch(lambda: torch.nn.functional.conv2d(x, w, stride=stride, padding=pad))
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
    cost_ms = t * 1e3
    return cost_ms, 2.0 * batch * Ho * Wo * OC * IC * kH * kW / 1e9 / cost_ms
