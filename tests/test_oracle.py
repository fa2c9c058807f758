"""CPU-only: the oracle against the golden vectors produced by the reference's host loops."""
import os

import numpy as np
import pytest

from tests import util

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _load(name):
    return np.load(os.path.join(GOLD, name))


def test_sgemm_naive_matches_reference_bits(oracle):
    g = _load("sgemm_ref.npz")
    names = sorted({k[:-2] for k in g.files})
    assert len(names) >= 6
    for n in names:
        c = oracle.sgemm_naive(g[n + "_a"], g[n + "_b"], fma=False)
        assert np.array_equal(c.view(np.uint32), g[n + "_c"].view(np.uint32)), n


def test_sgemm_known_answers(oracle):
    g = _load("sgemm_ref.npz")
    assert np.array_equal(g["s_id_c"], g["s_id_a"])
    assert np.all(g["s_one_c"] == 1000.0)
    assert np.all(oracle.sgemm_naive(g["s_one_a"], g["s_one_b"], fma=True) == 1000.0)


def test_hgemm_naive_matches_reference_bits(oracle):
    g = _load("hgemm_ref.npz")
    names = sorted({k.split("_a")[0] for k in g.files if k.endswith("_a")})
    assert len(names) >= 6
    for n in names:
        a, b_kn = g[n + "_a"], g[n + "_b_kn"]
        c16, _ = oracle.hgemm_naive(a, b_kn, b_is_nk=False)
        assert np.array_equal(c16.view(np.uint16), g[n + "_c"].view(np.uint16)), n
        c16t, _ = oracle.hgemm_naive(a, np.ascontiguousarray(b_kn.T), b_is_nk=True)
        assert np.array_equal(c16t.view(np.uint16), g[n + "_c"].view(np.uint16)), n


def test_hgemm_one_hot_is_exact(oracle):
    g = _load("hgemm_ref.npz")
    want = g["h_hot_b_kn"][np.arange(8) * 7]
    assert np.array_equal(g["h_hot_c"], want)


def test_conv_matches_reference_composition(oracle):
    """NHWC oracle vs reference im2col(NCHW)+cpuF16F16Gemm: same sums in another order."""
    g = _load("conv_ref.npz")
    for i in range(6):       # the last two: the 3-channel 7 x 7 / 2 first layer, and 3 x 3 at 64 -> 64 channels
        B, C, H, W, OC, kh, kw, stride, pad = (int(v) for v in g[f"c{i}_geom"])
        x = np.ascontiguousarray(g[f"c{i}_x_nchw"].transpose(0, 2, 3, 1))
        w = np.ascontiguousarray(g[f"c{i}_w_oihw"].transpose(0, 2, 3, 1))
        y16, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
        assert y16.shape == g[f"c{i}_y_nhwc"].shape
        util.assert_f16_close(g[f"c{i}_y_nhwc"], y32, f"conv case {i}")
        # half rounding of nearly equal fp32 sums differs by at most one ulp of the larger binade; the sums themselves
        # differ by the order of their fp32 additions, a few units of 2^-24 of the sum of the terms' magnitudes
        d = np.abs(y16.astype(np.float32) - g[f"c{i}_y_nhwc"].astype(np.float32))
        _, mag = oracle.conv2d_nhwc_f16(np.abs(x), np.abs(w), stride, pad)
        assert np.all(d <= 2 * np.spacing(np.abs(y16)).astype(np.float32) + 8 * 2.0 ** -24 * mag + 1e-7)
        assert np.mean(y16 != g[f"c{i}_y_nhwc"]) < 0.02


def test_live_reference_when_built(oracle):
    from oracle import ref
    if not ref.available():
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(5)
    a = rng.uniform(-1, 1, (50, 77)).astype(np.float32)
    b = rng.uniform(-1, 1, (77, 31)).astype(np.float32)
    assert np.array_equal(ref.cpuSgemm(a, b), oracle.sgemm_naive(a, b))
    ah, bh = a.astype(np.float16), b.astype(np.float16)
    assert np.array_equal(ref.cpuF16F16Gemm(ah, bh), oracle.hgemm_naive(ah, bh, b_is_nk=False)[0])


@pytest.mark.parametrize("tiling", [(6, 1, 16, 1, 4), (4, 1, 32, 1, 2), (2, 1, 16, 3, 1), (9, 1, 64, 1, 6)])
def test_template_nest_equals_definition(oracle, tiling):
    """The register-blocked loop nest keeps k ascending per output: bit-identical to the plain loop."""
    m1, m2, n1, n2, k1 = tiling
    rng = np.random.default_rng(11)
    M, N, K = 20 * m1 * m2, n1 * n2 * 2, 16 * k1
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    for fma in (False, True):
        assert np.array_equal(oracle.sgemm_template(a, b, m1, m2, n1, n2, k1, fma=fma),
                              oracle.sgemm_naive(a, b, fma=fma))


@pytest.mark.parametrize("shape", [(1, 1, 1), (130, 77, 101), (64, 256, 64), (7, 300, 33)])
def test_parallel_schedule_equals_definition(oracle, shape):
    M, N, K = shape
    rng = np.random.default_rng(12)
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    for threads in (1, 3):
        got = oracle.sgemm_parallel(a, b, tiling=(6, 1, 4, 16, 1, 2, 4), threads=threads)
        assert np.array_equal(got, oracle.sgemm_naive(a, b))


def test_fma_and_f64_variants_within_fp32_tolerance(oracle):
    from helix_b200 import datagen
    a, b = datagen.c1_fp32_gemm(256, 256, 1024)
    ref64 = oracle.sgemm_f64acc(a, b)
    for fma in (False, True):
        util.assert_f32_close(oracle.sgemm_naive(a, b, fma=fma), ref64, f"fma={fma}")


def test_fast_hgemm_within_tolerance(oracle):
    from helix_b200 import datagen
    a, b = datagen.c3_gemm(96, 200, 1000)
    f16, f32 = oracle.hgemm_fast(a, b)
    n16, n32 = oracle.hgemm_naive(a, b)
    util.assert_f16_close(f16, n32, "hgemm_fast")
    assert util.rel_fro(f32, n32) < 1e-6


def test_im2col_plus_gemm_equals_direct_conv(oracle):
    """Reference composition in fp32: im2col (NCHW) then GEMM == direct NHWC convolution."""
    rng = np.random.default_rng(3)
    B, C, H, W, OC, k, stride, pad = 2, 4, 7, 9, 5, 3, 2, 1
    x = rng.uniform(-1, 1, (B, C, H, W)).astype(np.float32)
    w = rng.standard_normal((OC, C, k, k)).astype(np.float32)
    col = oracle.im2col_nchw_f32(x, k, stride, pad)
    Ho, Wo = col.shape[2:]
    a = np.ascontiguousarray(col.transpose(0, 2, 3, 1).reshape(B * Ho * Wo, C * k * k))
    y_ref = oracle.sgemm_f64acc(a, np.ascontiguousarray(w.reshape(OC, -1).T)).reshape(B, Ho, Wo, OC)
    y = oracle.conv2d_nhwc_f32(np.ascontiguousarray(x.transpose(0, 2, 3, 1)),
                               np.ascontiguousarray(w.transpose(0, 2, 3, 1)), stride, pad)
    util.assert_f32_close(y, y_ref, "conv f32")


def test_half_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(9)
    v = (rng.standard_normal(4096) * 10.0 ** rng.integers(-6, 5, 4096)).astype(np.float32)
    assert np.array_equal(oracle.f32_to_f16(v).view(np.uint16), v.astype(np.float16).view(np.uint16))


def test_gemv_f32_lane_tree_is_a_reordering_of_the_plain_sum(oracle):
    """The 32-lane summation order of the fp32 GEMV stays within fp32 reassociation noise of the plain fmaf chain
    and of the fp64-accumulated product; with K <= 4 (one lane holds everything) it IS the plain chain."""
    rng = np.random.default_rng(5)
    w = rng.uniform(-1, 1, (37, 1000)).astype(np.float32)
    x = rng.uniform(-1, 1, (3, 1000)).astype(np.float32)
    y = oracle.gemv_f32_lane_tree(w, x)
    ref64 = (x.astype(np.float64) @ w.astype(np.float64).T)
    assert np.linalg.norm(y - ref64) / np.linalg.norm(ref64) <= 1e-6
    chain = oracle.sgemm_naive(x, np.ascontiguousarray(w.T), fma=True)
    assert np.linalg.norm(y - chain) / np.linalg.norm(chain) <= 1e-6
    w4, x4 = w[:, :4].copy(), x[:, :4].copy()
    assert np.array_equal(oracle.gemv_f32_lane_tree(w4, x4), oracle.sgemm_naive(x4, np.ascontiguousarray(w4.T), fma=True))
