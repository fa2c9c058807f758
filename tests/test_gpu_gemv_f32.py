"""GPU tests of the true-fp32 GEMV (helix_gemv_f32): bit-exact against the oracle's restatement of its
summation order, within 1e-5 of the fp64-accumulated product, every compiled variant, split-K deterministic."""
import numpy as np
import pytest
import torch

from helix_b200 import ops
from helix_b200._lib import OP_GEMV_F32
from tests import util

pytestmark = pytest.mark.gpu


def _data(rows, K, m, seed):
    rng = np.random.default_rng(seed)
    w = rng.uniform(-1, 1, (rows, K)).astype(np.float32)
    x = rng.uniform(-1, 1, (m, K)).astype(np.float32)
    return w, x


@pytest.mark.parametrize("rows,K,m", [(4096, 4096, 1), (1000, 1028, 2), (333, 516, 3), (64, 128, 8), (5, 8, 5),
                                      (2050, 4100, 4)])
def test_gemv_f32_is_bit_exact_in_its_stated_order(oracle, rows, K, m):
    w, x = _data(rows, K, m, rows + K + m)
    want = oracle.gemv_f32_lane_tree(w, x)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    got = ops.gemv_f32(wd, xd).cpu().numpy()
    assert np.array_equal(got, want)
    # every compiled (rows per warp, loads in flight) variant sums in the same order
    for rpw in (1, 2):
        for unroll in (2, 4, 8):
            if rpw == 2 and unroll == 8:
                continue
            cfg = ops.make_cfg(OP_GEMV_F32, tile_m=1, tile_n=rpw, tile_k=128, split_k=1, load_group=unroll)
            assert np.array_equal(ops.gemv_f32(wd, xd, cfg=cfg).cpu().numpy(), want), (rpw, unroll)
    ref64 = x.astype(np.float64) @ w.astype(np.float64).T
    util.assert_f32_close(got, ref64, f"fp32 GEMV {rows}x{K} m={m}")
    # transposed output layout
    out_t = torch.empty((rows, m), dtype=torch.float32, device="cuda")
    ops.run(ops.launch_gemv_f32(wd, xd, out_t, out_transposed=True))
    torch.cuda.synchronize()
    assert np.array_equal(out_t.cpu().numpy().T, want)
    ops.check_status()


def test_gemv_f32_split_k_is_deterministic_and_close(oracle):
    rows, K, m = 96, 16384, 2
    w, x = _data(rows, K, m, 3)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    cfg = ops.make_cfg(OP_GEMV_F32, tile_m=1, tile_n=2, tile_k=128, split_k=4, load_group=4)
    a = ops.gemv_f32(wd, xd, cfg=cfg).cpu().numpy()
    b = ops.gemv_f32(wd, xd, cfg=cfg).cpu().numpy()
    assert np.array_equal(a, b)
    # slice sums in slice order: the oracle's order applied per slice, then added in sequence
    want = np.zeros((m, rows), np.float32)
    for s in range(4):
        want = want + oracle.gemv_f32_lane_tree(np.ascontiguousarray(w[:, s * 4096:(s + 1) * 4096]),
                                                np.ascontiguousarray(x[:, s * 4096:(s + 1) * 4096]))
    assert np.array_equal(a, want)
    auto = ops.gemv_f32(wd, xd).cpu().numpy()       # the library's own split for few rows and a long K
    util.assert_f32_close(auto, x.astype(np.float64) @ w.astype(np.float64).T, "fp32 GEMV automatic split")
    ops.check_status()


def test_gemv_f32_rejects_unaligned_k():
    w = torch.zeros((8, 6), dtype=torch.float32, device="cuda")
    x = torch.zeros((1, 6), dtype=torch.float32, device="cuda")
    with pytest.raises(Exception) as e:
        ops.gemv_f32(w, x)
    assert "-2" in str(e.value)
