"""GPU test of the failure path every kernel shares: a bounded wait that runs out reports HELIX_ERR_TIMEOUT
through the status word and the kernel returns; the context stays usable."""
import time

import numpy as np
import pytest
import torch

from helix_b200 import _lib, datagen, ops

pytestmark = pytest.mark.gpu


def test_a_wait_that_nothing_satisfies_gives_up_and_reports_a_timeout(oracle):
    ops.check_status()                                   # clean before
    t0 = time.perf_counter()
    ops.selftest_bounded_wait(3_000_000)                 # 3 ms limit on a barrier nobody arrives at
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0                # the kernel returned by itself
    with pytest.raises(_lib.HelixError) as e:
        ops.check_status()
    assert e.value.status == -5 and "wait ran out" in str(e.value)
    ops.check_status()                                   # reading the word cleared it
    # the context is intact: the next product launch runs and is right
    a, b = datagen.c3_gemm(256, 192, 320, seed=8)
    c = ops.gemm_f16(torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
    torch.cuda.synchronize()
    ops.check_status()
    _, ref = oracle.hgemm_naive(a, b)
    assert np.linalg.norm(c.cpu().numpy().astype(np.float64) - ref) / np.linalg.norm(ref) <= 2e-3


def test_the_self_test_validates_its_arguments(lib):
    import ctypes
    w = ops.status_word()
    assert lib.helix_selftest_bounded_wait(0, ctypes.c_void_p(w.data_ptr()), None) == -1
    assert lib.helix_selftest_bounded_wait(2_000_000_000, ctypes.c_void_p(w.data_ptr()), None) == -1
    assert lib.helix_selftest_bounded_wait(1000, None, None) == -1
