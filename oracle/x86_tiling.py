"""Restatement of the reference's x86 profile and tiling chooser.  Test infrastructure only.

The reference measures 270 register-block candidates of its single-thread template
(scripts/x86_CPU/profile_x86_CPU.py:62-91), extends the fast ones to cache blocks of up to 256 x 256
outputs (:93-117), stores {(M, N, K) cache block: (register block, seconds, GFLOP/s)}, and picks per
problem the cache block minimising seconds x row blocks x waves of column panels over the threads
(scripts/x86_CPU/benchmark_x86_CPU_gemm.py:46-68, the same function in x86_CPU_runtime_cost.py:40-62).
Here the candidates are timed on the C restatement of that template (oracle_sgemm_template), since the
TVM tool chain that generates the reference's code is not available.

Two reference quirks are not reproduced: the cache-block cost is the probe's cost scaled by the number
of micro-kernel cells it really holds (the probe has 20 row blocks of one column block; the reference
divides by 20 * 16, which makes its own 60 % filter pass everything), and the K extent of a padded
problem is ceil(K / k1) * k1 (x86_CPU_runtime_cost.py:72 drops the factor k1).
"""
import ctypes
import math

from . import api

PEAK_GFLOPS = 153.0        # the reference's per-core peak (profile_x86_CPU.py:14)
KEEP_FRACTION = 0.6        # candidates below this share of the peak are dropped (:90, :113)
PROBE_ROW_BLOCKS = 20      # the probe problem is M = 20 * m1 rows (:77)


def probe_grid():
    """(m1, m2, n1, n2, k1) of the 270 probes in the reference's loop order (profile_x86_CPU.py:70-79)."""
    out = []
    for M1 in range(1, 10):
        for N1 in range(1, 6):
            for K1 in range(1, 7):
                n1, n2 = (16, N1) if N1 in (3, 5) else (N1 * 16, 1)
                out.append((M1, 1, n1, n2, K1))
    return out


def time_probe(m1, m2, n1, n2, k1, fma=True, min_seconds=2e-3):
    """Seconds per call of the single-thread template on the reference's probe problem
    (M = 20 * m1 * m2, N = n1 * n2, K = 16 * k1)."""
    lib = api.lib()
    lib.oracle_time_sgemm_template.restype = ctypes.c_double
    lib.oracle_time_sgemm_template.argtypes = [ctypes.c_int] * 9 + [ctypes.c_double]
    M, N, K = m1 * m2 * PROBE_ROW_BLOCKS, n1 * n2, k1 * 16
    t = lib.oracle_time_sgemm_template(M, N, K, m1, m2, n1, n2, k1, int(fma), float(min_seconds))
    if t <= 0:
        raise RuntimeError("oracle_time_sgemm_template failed")
    return t


def register_blocks(timer=time_probe, peak=PEAK_GFLOPS, keep=KEEP_FRACTION):
    """{(m1*m2, n1*n2, k1): (seconds, GFLOP/s)} of the probes faster than keep * peak, and the best GFLOP/s
    seen.  When no probe reaches keep * peak (the C restatement on this host is slower than the
    generated code the reference's 153 GFLOP/s refers to) the threshold is taken relative to the best
    probe instead, so the dictionary is never empty."""
    seen = {}
    for (m1, m2, n1, n2, k1) in probe_grid():
        M, N, K = m1 * m2 * PROBE_ROW_BLOCKS, n1 * n2, k1 * 16
        cost = timer(m1, m2, n1, n2, k1)
        seen[(m1 * m2, n1 * n2, k1)] = (cost, 2.0 * M * N * K * 1e-9 / cost)
    best = max(v[1] for v in seen.values())
    used_peak = peak if best > keep * peak else best
    kept = {k: v for k, v in seen.items() if v[1] > keep * used_peak or v[1] == best}
    return kept, best, used_peak


def cache_blocks(reg, peak, keep=KEEP_FRACTION, limit=256):
    """Extend register blocks to cache blocks of up to limit x limit outputs (profile_x86_CPU.py:93-117):
    {(M, N, K): (register block, seconds, GFLOP/s)} keeping, per block, the fastest register block."""
    out = {}
    for key, (cost, _) in reg.items():
        m1, n1, k1 = key
        for mx in range(1, limit // m1 + 1):
            for nx in range(1, limit // n1 + 1):
                M, N, K = mx * m1, nx * n1, 16 * k1
                c = cost / PROBE_ROW_BLOCKS * (mx * nx)      # the probe holds 20 cells of this register block
                f = 2.0 * M * N * K * 1e-9 / c
                if f > keep * peak and ((M, N, K) not in out or out[(M, N, K)][1] > c):
                    out[(M, N, K)] = (key, c, f)
    return out


def profile(timer=time_probe, peak=PEAK_GFLOPS, keep=KEEP_FRACTION):
    """The dictionary the reference writes to build/prof_dict/x86_CPU_cost_model.dict, plus what the
    threshold was taken against."""
    reg, best, used_peak = register_blocks(timer, peak, keep)
    return cache_blocks(reg, used_peak, keep), {"best_probe_gflops": best, "threshold_peak_gflops": used_peak,
                                                "reference_peak_gflops": peak, "register_blocks_kept": len(reg)}


def get_tiling(prof_dict, M, N, K, threads):
    """(m1, m2, m3, n1, n2, n3, k1) for the parallel packed schedule, chosen as benchmark_x86_CPU_gemm.py:46-68
    does: cost = seconds(cache block) * ceil(M / Mc) * ceil(ceil(N / Nc) / threads); first minimum wins."""
    min_cost, min_cache, min_reg = float("inf"), (1, 1, 1), (1, 1, 1)
    for k, v in prof_dict.items():
        panels = math.ceil(N / k[1])
        cost = v[1] * math.ceil(M / k[0]) * math.ceil(panels / threads)
        if min_cost > cost:
            min_cost, min_cache, min_reg = cost, k, v[0]
    m1, m2, m3 = min_reg[0], 1, min_cache[0] // min_reg[0]
    n1, n2, n3 = min_reg[1], 1, min_cache[1] // min_reg[1]
    if n1 in (48, 80):
        n2, n1 = n1 // 16, 16
    return m1, m2, m3, n1, n2, n3, min_reg[2]


def padded_extents(M, N, K, tiling):
    """Extents the schedule really runs: every axis rounded up to its tile (benchmark_x86_CPU_gemm.py:78,117)."""
    m1, m2, m3, n1, n2, n3, k1 = tiling
    mc, nc = m1 * m2 * m3, n1 * n2 * n3
    return math.ceil(M / mc) * mc, math.ceil(N / nc) * nc, math.ceil(K / k1) * k1
