"""GPU parity: true-fp32 SIMT GEMM through the C ABI vs the CPU oracle (bit-exact vs an fmaf chain)."""
import os

import numpy as np
import pytest
import torch

from helix_b200 import datagen, ops
from helix_b200._lib import OP_GEMM_F32
from tests import util

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _run(a, b, trans_a=False, cfg=None):
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    M = a.shape[1] if trans_a else a.shape[0]
    out = torch.full((M, b.shape[1]), float("nan"), dtype=torch.float32, device="cuda")
    ops.run(ops.launch_gemm_f32(ad, bd, out, trans_a, cfg))
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("cfg_idx", range(10))
@pytest.mark.parametrize("shape", [(128, 128, 64), (257, 131, 67), (1, 1, 1), (64, 300, 1000), (5, 1024, 16),
                                   (260, 392, 8), (132, 136, 200)])
def test_sgemm_bit_exact_vs_fma_chain(oracle, shape, cfg_idx):
    M, N, K = shape
    a, b = datagen.c1_fp32_gemm(M, N, K, seed=10 + cfg_idx)
    cfg = ops.configs(OP_GEMM_F32)[cfg_idx]
    got = _run(a, b, cfg=cfg)
    want = oracle.sgemm_naive(a, b, fma=True)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (shape, cfg.key())


def test_sgemm_config1_1024_cubed(oracle):
    """FP32 GEMM 1024^3, U[-1,1], seed 0: within 1e-5 of the reference-style loop, bit-equal to the FMA chain."""
    a, b = datagen.c1_fp32_gemm()
    got = _run(a, b)
    assert np.array_equal(got, oracle.sgemm_naive(a, b, fma=True))
    util.assert_f32_close(got, oracle.sgemm_parallel(a, b), "vs parallel template (mul+add)")
    util.assert_f32_close(got, oracle.sgemm_f64acc(a, b), "vs fp64 accumulate")


@pytest.mark.parametrize("trans_a", [False, True])
@pytest.mark.parametrize("cfg_idx", range(5))
def test_sgemm_pipelined_kernel_ragged_sizes_inside_aligned_leading_dimensions(oracle, cfg_idx, trans_a):
    """16-byte-aligned rows but M, N, K that are not multiples of 4: the cp.async ring zero-fills partial
    chunks at the K and N tails and whole chunks outside M; the result stays the fmaf chain, bit for bit."""
    cfg = ops.configs(OP_GEMM_F32)[cfg_idx]
    assert cfg.stages >= 3
    M, N, K = 203, 262, 150 + cfg_idx
    a, b = datagen.c1_fp32_gemm(M, N, K, seed=30 + cfg_idx)
    want = oracle.sgemm_naive(a, b, fma=True)
    big_a = torch.full((K + 3, 208) if trans_a else (M + 1, 160), float("nan"), device="cuda")
    big_b = torch.full((K + 2, 264), float("nan"), device="cuda")
    big_c = torch.full((M + 1, 272), -7.0, device="cuda")
    av = big_a[:K, :M] if trans_a else big_a[:M, :K]
    av.copy_(torch.from_numpy(np.ascontiguousarray(a.T) if trans_a else a))
    big_b[:K, :N].copy_(torch.from_numpy(b))
    ops.run(ops.launch_gemm_f32(av, big_b[:K, :N], big_c[:M, :N], trans_a, cfg))
    torch.cuda.synchronize()
    ops.check_status()
    got = big_c.cpu().numpy()
    assert np.array_equal(got[:M, :N].view(np.uint32), want.view(np.uint32))
    assert np.all(got[M:] == -7.0) and np.all(got[:, N:] == -7.0)       # nothing written outside C


def test_sgemm_transposed_a_layout(oracle):
    a, b = datagen.c1_fp32_gemm(200, 96, 130, seed=4)
    got = _run(np.ascontiguousarray(a.T), b, trans_a=True)
    assert np.array_equal(got, oracle.sgemm_naive(a, b, fma=True))


def test_sgemm_unaligned_leading_dimensions(oracle):
    a, b = datagen.c1_fp32_gemm(70, 33, 45, seed=5)   # N, K not multiples of 4: scalar path
    got = _run(a, b)
    assert np.array_equal(got, oracle.sgemm_naive(a, b, fma=True))


def test_sgemm_golden_vectors_from_reference_loop():
    g = np.load(os.path.join(GOLD, "sgemm_ref.npz"))
    for n in sorted({k[:-2] for k in g.files}):
        got = _run(g[n + "_a"], g[n + "_b"])
        util.assert_f32_close(got, g[n + "_c"], n)
    assert np.all(_run(g["s_one_a"], g["s_one_b"]) == 1000.0)
    assert np.array_equal(_run(g["s_id_a"], g["s_id_b"]), g["s_id_a"])
