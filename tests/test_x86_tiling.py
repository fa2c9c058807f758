"""CPU tests of the restated x86 profile and tiling chooser (oracle/x86_tiling.py) and of the
register-resident micro-kernel the timed CPU baseline runs."""
import math

import numpy as np
import pytest

from oracle import x86_tiling as xt


def test_probe_grid_is_the_references_270_candidates():
    grid = xt.probe_grid()
    assert len(grid) == 9 * 5 * 6
    # N1 = 3 and 5 become three / five 16-wide column blocks (profile_x86_CPU.py:75-77)
    assert (4, 1, 16, 3, 2) in grid and (4, 1, 16, 5, 2) in grid and (4, 1, 64, 1, 2) in grid
    assert {(m1 * m2, n1 * n2, k1) for m1, m2, n1, n2, k1 in grid} == \
        {(m, n, k) for m in range(1, 10) for n in (16, 32, 48, 64, 80) for k in range(1, 7)}


def _fake_timer(rate_of):
    def timer(m1, m2, n1, n2, k1):
        M, N, K = m1 * m2 * 20, n1 * n2, k1 * 16
        return 2.0 * M * N * K * 1e-9 / rate_of(m1 * m2, n1 * n2, k1)
    return timer


def test_register_blocks_keep_what_beats_sixty_percent_of_the_peak():
    # a machine on which only 8 x 64 blocks are fast
    timer = _fake_timer(lambda m, n, k: 120.0 if (m, n) == (8, 64) else 40.0)
    reg, best, used = xt.register_blocks(timer)
    assert used == xt.PEAK_GFLOPS and best == pytest.approx(120.0)
    assert set(reg) == {(8, 64, k) for k in range(1, 7)}
    # nothing reaches the reference's threshold: the threshold moves to the best probe, the dictionary is not empty
    reg2, best2, used2 = xt.register_blocks(_fake_timer(lambda m, n, k: 10.0 + m))
    assert used2 == pytest.approx(19.0) and best2 == pytest.approx(19.0)
    assert reg2 and all(v[1] > 0.6 * 19.0 or v[1] == best2 for v in reg2.values())


def test_cache_blocks_scale_the_probe_by_its_twenty_cells():
    cost = 1e-6
    blocks = xt.cache_blocks({(8, 64, 2): (cost, 130.0)}, peak=1.0)
    # the probe is 20 row blocks of one column block: one cell costs cost / 20
    assert blocks[(8, 64, 32)][1] == pytest.approx(cost / 20)
    assert blocks[(16, 128, 32)][1] == pytest.approx(cost / 20 * 4)
    assert max(k[0] for k in blocks) <= 256 and max(k[1] for k in blocks) <= 256
    assert all(v[0] == (8, 64, 2) for v in blocks.values())
    # the 60 % filter is a real filter here: a slow register block yields no cache block
    assert xt.cache_blocks({(8, 64, 2): (1.0, 0.001)}, peak=153.0) == {}


def test_get_tiling_follows_the_references_cost_formula():
    prof = {
        (64, 64, 32): ((8, 64, 2), 4.0e-6, 100.0),
        (128, 256, 32): ((8, 64, 2), 30.0e-6, 110.0),
        (90, 48, 16): ((9, 48, 1), 3.0e-6, 95.0),
    }
    M, N, K, threads = 1000, 1000, 512, 8

    def cost(k):
        return prof[k][1] * math.ceil(M / k[0]) * math.ceil(math.ceil(N / k[1]) / threads)
    best = min(prof, key=cost)
    tl = xt.get_tiling(prof, M, N, K, threads)
    reg = prof[best][0]
    assert tl[0] == reg[0] and tl[2] == best[0] // reg[0] and tl[6] == reg[2]
    # a 48-wide register block is three 16-wide vectors (benchmark_x86_CPU_gemm.py:63-65)
    tl48 = xt.get_tiling({(90, 48, 16): prof[(90, 48, 16)]}, M, N, K, threads)
    assert tl48 == (9, 1, 10, 16, 3, 1, 1)
    assert xt.padded_extents(1000, 1000, 500, tl48) == (1080, 1008, 500)


@pytest.mark.parametrize("fma", [True, False])
@pytest.mark.parametrize("shape", [(130, 200, 77), (64, 64, 64), (257, 96, 300)])
def test_chosen_tiling_is_bit_equal_to_the_plain_loop(oracle, shape, fma):
    """Whatever tiling the chooser returns for a ragged problem, the parallel packed schedule (register
    resident micro-kernel included) reproduces the plain k-ascending loop bit for bit."""
    prof = xt.cache_blocks({(6, 64, 1): (1e-6, 120.0), (8, 32, 2): (1.2e-6, 110.0), (9, 48, 3): (2e-6, 100.0),
                            (4, 80, 1): (1e-6, 100.0)}, peak=1.0)
    M, N, K = shape
    rng = np.random.default_rng(sum(shape))
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    want = oracle.sgemm_naive(a, b, fma=fma)
    for threads in (1, 3):
        tl = xt.get_tiling(prof, M, N, K, threads)
        assert np.array_equal(oracle.sgemm_parallel(a, b, tiling=tl, threads=threads, fma=fma), want), tl
    for tl in [(9, 1, 2, 16, 3, 1, 2), (4, 1, 1, 16, 5, 2, 1), (8, 2, 2, 64, 1, 1, 4), (5, 1, 1, 48, 1, 1, 6)]:
        assert np.array_equal(oracle.sgemm_parallel(a, b, tiling=tl, threads=2, fma=fma), want), tl
    m1, n1, k1 = 5, 32, 4
    ap, bp = a[:M // m1 * m1, :K // k1 * k1], b[:K // k1 * k1, :N // n1 * n1]
    assert np.array_equal(oracle.sgemm_template(ap, bp, m1, 1, n1, 1, k1, fma=fma), oracle.sgemm_naive(ap, bp, fma=fma))


def test_profile_runs_on_this_host_and_picks_usable_tilings(oracle):
    prof, info = xt.profile()
    assert prof and info["register_blocks_kept"] >= 1 and info["best_probe_gflops"] > 0
    tl = xt.get_tiling(prof, 300, 500, 200, threads=4)
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (300, 200)).astype(np.float32)
    b = rng.uniform(-1, 1, (200, 500)).astype(np.float32)
    assert np.array_equal(oracle.sgemm_parallel(a, b, tiling=tl, threads=4, fma=True), oracle.sgemm_naive(a, b, fma=True))
