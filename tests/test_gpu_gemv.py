"""GPU parity: fp16 GEMV (1..8 right-hand sides) through the C ABI vs the CPU oracle."""
import numpy as np
import pytest
import torch

from helix_b200 import datagen, ops
from helix_b200._lib import OP_GEMV_F16
from tests import util

pytestmark = pytest.mark.gpu


def _run(w, x, cfg=None, transposed=False):
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    if transposed:
        out = torch.full((w.shape[0], x.shape[0]), float("nan"), dtype=torch.float16, device="cuda")
        ops.run(ops.launch_gemv_f16(wd, xd, out, cfg, out_transposed=True))
        res = out.t()
    else:
        out = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=torch.float16, device="cuda")
        ops.run(ops.launch_gemv_f16(wd, xd, out, cfg))
        res = out
    torch.cuda.synchronize()
    ops.check_status()
    return res.cpu().numpy()


@pytest.mark.parametrize("rows,K,m", [(4096, 4096, 1), (1000, 1024, 1), (7, 8, 1), (1, 256, 1), (129, 264, 2),
                                      (513, 2048, 3), (300, 4096, 4), (64, 512, 8), (4096, 4096, 8), (33, 40, 5)])
def test_gemv_matches_oracle(oracle, rows, K, m):
    w, x = datagen.c2_gemv(rows, K, m, seed=1)
    got = _run(w, x)
    _, ref32 = oracle.hgemm_naive(x, w)  # [m, rows]
    util.assert_f16_close(got, ref32, f"gemv {rows}x{K} m={m}")


@pytest.mark.parametrize("split", [2, 4, 16])
def test_gemv_split_k_is_deterministic_and_close(oracle, split):
    w, x = datagen.c2_gemv(96, 8192, 2, seed=7)
    cfg = ops.make_cfg(OP_GEMV_F16, tile_m=1, tile_n=2, tile_k=256, split_k=split)
    a = _run(w, x, cfg)
    b = _run(w, x, cfg)
    assert np.array_equal(a.view(np.uint16), b.view(np.uint16))
    _, ref32 = oracle.hgemm_naive(x, w)
    util.assert_f16_close(a, ref32, f"gemv split_k={split}")


def test_gemv_transposed_output_layout(oracle):
    """N <= 8 case of the reference sweep, e.g. (7680, 2, 2560): C[M, N] with the matrix on M."""
    w, x = datagen.c2_gemv(640, 2560, 2, seed=3)
    got = _run(w, x, transposed=True)
    _, ref32 = oracle.hgemm_naive(x, w)
    util.assert_f16_close(got, ref32, "gemv transposed")


def test_gemv_known_answer_ones():
    w = np.ones((50, 1024), np.float16)
    x = np.ones((1, 1024), np.float16)
    assert np.all(_run(w, x) == 1024.0)


def test_gemv_rejects_bad_arguments():
    w = torch.zeros((8, 20), dtype=torch.float16, device="cuda")   # K not a multiple of 8
    x = torch.zeros((1, 20), dtype=torch.float16, device="cuda")
    out = torch.zeros((1, 8), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception) as e:
        ops.run(ops.launch_gemv_f16(w, x, out))
    assert "-2" in str(e.value)
    x9 = torch.zeros((9, 24), dtype=torch.float16, device="cuda")
    w24 = torch.zeros((8, 24), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.run(ops.launch_gemv_f16(w24, x9, torch.zeros((9, 8), dtype=torch.float16, device="cuda")))


@pytest.mark.parametrize("flag", [1, 2])
def test_gemv_launch_ordering_flags_do_not_change_results(oracle, flag):
    """INDEPENDENT (1) and STATIC_A (2) only move the wait for the preceding kernel; a chain of launches on
    distinct outputs must give bit-identical results to fully ordered launches."""
    w, x = datagen.c2_gemv(2048, 4096, 1, seed=5)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    outs = [torch.full((1, 2048), float("nan"), dtype=torch.float16, device="cuda") for _ in range(6)]
    ref = ops.gemv_f16(wd, xd)
    for o in outs:
        l = ops.launch_gemv_f16(wd, xd, o)
        l.flags = flag
        ops.run(l)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, ref)
    _, ref32 = oracle.hgemm_naive(x, w)
    util.assert_f16_close(ref.cpu().numpy(), ref32, "gemv flags")
