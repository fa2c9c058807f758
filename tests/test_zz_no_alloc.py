"""GPU test of helix_gemv_f16_static, the split-K GEMV that never calls the device allocator.

The entry point exists for callers that are not in a position to allocate when they need the
product (all HBM already owned by their own pool): its split-K
partial sums go to a fixed array inside the library.  This file is named so that pytest collects
it after every other test file; it must pass both alone in a fresh process and at the end of a
full run, because the fixed array is shared by all calls and keeps whatever the last one left.
"""
import ctypes

import numpy as np
import pytest
import torch

from helix_b200 import _lib, datagen, ops
from helix_b200._lib import OP_GEMV_F16
from tests import util

pytestmark = pytest.mark.gpu


def _static(lib, w, x, split_k):
    out = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=torch.float16, device="cuda")
    rc = lib.helix_gemv_f16_static(w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0), out.data_ptr(),
                                   out.stride(0), 1, w.shape[0], w.shape[1], x.shape[0], split_k,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_scratch_gemv_matches_workspace_gemv_twice_in_a_row(lib, oracle):
    """Two consecutive calls with different shapes: the second starts with the first one's partials
    still in the shared array and must not be disturbed by them."""
    cases = [(1536, 4096, 3, 4), (700, 8192, 8, 8)]
    for rows, K, m, split in cases:
        wn, xn = datagen.c2_gemv(rows, K, m, seed=21)
        w, x = torch.from_numpy(wn).cuda(), torch.from_numpy(xn).cuda()
        out = torch.full((m, rows), float("nan"), dtype=torch.float16, device="cuda")
        _static(lib, w, x, split)                     # first call on this device: does the symbol look-up
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        rc = lib.helix_gemv_f16_static(w.data_ptr(), w.stride(0), x.data_ptr(), x.stride(0), out.data_ptr(),
                                       out.stride(0), 1, rows, K, m, split,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0
        # the point of the entry point: the call took no device memory, from the driver or from torch
        assert free_after == free_before and torch.cuda.memory_allocated() == torch_before
        got = out
        cfg = ops.make_cfg(OP_GEMV_F16, tile_m=1, tile_n=(2 if m <= 2 else 1), tile_k=256, split_k=split,
                           load_group=(4 if m <= 4 else 2))
        want = ops.gemv_f16(w, x, cfg=cfg)            # the existing entry point, caller workspace
        torch.cuda.synchronize()
        got_n, want_n = got.cpu().numpy(), want.cpu().numpy()
        # same kernel, same slices, same summation order: the two entry points agree bit for bit
        assert np.array_equal(got_n.view(np.uint16), want_n.view(np.uint16)), f"static vs workspace GEMV {rows}x{K} m={m}"
        _, ref32 = oracle.hgemm_naive(xn, wn)
        util.assert_f16_close(got_n, ref32, f"static GEMV vs oracle {rows}x{K} m={m}")


def test_static_scratch_gemv_rejects_what_does_not_fit(lib):
    rows, K, m, split = 1 << 17, 4096, 8, 2          # 2 * 8 * 131072 floats > 1 Mi floats
    w = torch.zeros((8, K), dtype=torch.float16, device="cuda")   # never dereferenced: rejected first
    x = torch.zeros((m, K), dtype=torch.float16, device="cuda")
    y = torch.zeros((m, 8), dtype=torch.float16, device="cuda")
    rc = lib.helix_gemv_f16_static(w.data_ptr(), K, x.data_ptr(), K, y.data_ptr(), rows, 1, rows, K, m, split, None)
    assert rc == -8
    assert b"capacity" in lib.helix_status_string(rc)


def test_static_scratch_gemv_single_pass_is_never_rejected_for_size(lib, oracle):
    """split_k = 1 (asked for, or what a short K is clamped to) does not use the array: no capacity limit."""
    rows, K, m = 200000, 256, 8                       # 8 * 200000 floats > 1 Mi floats
    wn, xn = datagen.c2_gemv(rows, K, m, seed=5)
    w, x = torch.from_numpy(wn).cuda(), torch.from_numpy(xn).cuda()
    for split in (1, 4):                              # 4 slices of 64 < 256 elements: runs as one pass
        rc, got = _static(lib, w, x, split)
        torch.cuda.synchronize()
        assert rc == 0
        _, ref32 = oracle.hgemm_naive(xn[:, :], wn[:4096])
        util.assert_f16_close(got.cpu().numpy()[:, :4096], ref32, f"single-pass static GEMV split={split}")
