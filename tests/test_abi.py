"""CPU-only: the C-ABI library loads, exports every declared symbol, and validates arguments."""
import ctypes
import os
import re

from helix_b200 import _lib
from helix_b200._lib import Cfg, DevInfo, Launch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "helix_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(helix_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(lib):
    names = declared_symbols()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/helix_b200.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) == set(names)


def test_struct_sizes_match_header_layout():
    # helix_cfg_t: 16 ints; helix_devinfo_t: 5 ints (+pad) + 4 int64 + 64 chars
    assert ctypes.sizeof(Cfg) == 64
    assert ctypes.sizeof(DevInfo) == 24 + 32 + 64
    assert Launch.cfg.offset == 4 and Launch.a.offset == 72


def test_version_and_status_strings(lib):
    assert lib.helix_version() >= 100
    for code in range(0, -8, -1):
        assert lib.helix_status_string(code)
    assert lib.helix_status_string(-5) == b"bounded device-side wait ran out"


def test_config_enumeration(lib):
    for op in (_lib.OP_GEMM_F16, _lib.OP_GEMV_F16, _lib.OP_CONV_F16, _lib.OP_GEMM_F32, _lib.OP_CONV_F32):
        n = lib.helix_num_configs(op)
        assert n > 0
        seen = set()
        for i in range(n):
            c = Cfg()
            rc = lib.helix_get_config(op, i, ctypes.byref(c))
            if rc == 0:
                assert c.op == op and c.tile_m > 0 and c.split_k >= 1
                seen.add((c.key(), c.thread_m, c.thread_n))
        assert len(seen) >= 3
        assert lib.helix_get_config(op, n, ctypes.byref(Cfg())) == -1
    assert lib.helix_num_configs(99) == -1


def test_default_config_and_workspace_are_consistent(lib):
    for (M, N, K, b) in [(4096, 4096, 4096, 1), (16, 11008, 4096, 1), (128, 4096, 11008, 1), (512, 512, 64, 192)]:
        l = Launch()
        l.op, l.M, l.N, l.K, l.batch = _lib.OP_GEMM_F16, M, N, K, b
        c = Cfg()
        assert lib.helix_default_config(ctypes.byref(l), ctypes.byref(c)) == 0
        assert c.tile_m == 128 and c.tile_n in (16, 32, 64, 128, 256) and c.stages >= 2
        ws = lib.helix_workspace_bytes(ctypes.byref(l))
        if c.stream_k:
            pm, pn = (N, M) if c.swap_ab else (M, N)
            tiles = -(-pm // 128) * -(-pn // c.tile_n) * b
            grid = min(tiles * -(-K // 64), 148)   # no device here: the library assumes 148 SMs
            assert ws == (0 if tiles % grid == 0 else 2 * grid * 128 * c.tile_n * 4)
        elif c.split_k == 1:
            assert ws == 0
        else:
            # split-K: one 8-byte arrival counter per tile (rounded up to 1 KiB), then one 128 x tile_n fp32 slot
            # per tile and slice
            pm, pn = (N, M) if c.swap_ab else (M, N)
            tiles = -(-pm // 128) * -(-pn // c.tile_n) * b
            assert ws == -(-tiles * 8 // 1024) * 1024 + tiles * c.split_k * 128 * c.tile_n * 4


def test_launch_without_device_reports_nodevice_or_runs(lib):
    """No compute here: with no GPU the launch entry points return HELIX_ERR_NODEVICE, never crash."""
    import torch
    if torch.cuda.is_available():
        return
    l = Launch()
    l.op, l.M, l.N, l.K, l.batch = _lib.OP_GEMM_F16, 128, 128, 64, 1
    assert lib.helix_launch(ctypes.byref(l), None, None) == -7
    assert lib.helix_launch(None, None, None) == -1


def test_conv_f32_workspace_is_column_matrix_plus_transposed_weights(lib):
    l = Launch()
    l.op = _lib.OP_CONV_F32
    for i, v in enumerate((2, 10, 10, 8, 16, 3, 3, 1, 1)):      # N H W C KO R S stride pad
        l.conv[i] = v
    M, K = 2 * 10 * 10, 3 * 3 * 8
    need = lib.helix_workspace_bytes(ctypes.byref(l))
    assert need % 256 == 0 and (M * K + K * 16) * 4 <= need <= (M * K + K * 16) * 4 + 512
    for i, v in enumerate((1, 6, 6, 8, 4, 1, 1, 1, 0)):          # 1x1: no column matrix
        l.conv[i] = v
    assert lib.helix_workspace_bytes(ctypes.byref(l)) == 256
    c = Cfg()
    assert lib.helix_default_config(ctypes.byref(l), ctypes.byref(c)) == 0 and c.op == _lib.OP_CONV_F32 and c.tile_m > 0
