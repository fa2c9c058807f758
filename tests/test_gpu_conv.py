"""GPU parity: implicit-GEMM NHWC convolution through the C ABI vs the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from helix_b200 import datagen, ops
from helix_b200._lib import OP_CONV_F16
from tests import util

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _run(x, w, stride, pad, cfg=None):
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    out = ops.conv2d_f16_nhwc(xd, wd, stride, pad, cfg=cfg)
    torch.cuda.synchronize()
    ops.check_status()
    return out.cpu().numpy()


@pytest.mark.parametrize("geom", [
    (2, 8, 9, 9, 16, 3, 3, 1, 1), (1, 16, 12, 10, 8, 3, 3, 2, 1), (2, 8, 6, 6, 8, 1, 1, 1, 0),
    (1, 8, 11, 11, 8, 5, 5, 2, 2), (3, 64, 14, 14, 64, 3, 3, 1, 1), (2, 24, 17, 13, 40, 3, 3, 1, 0),
    (2, 64, 8, 8, 32, 1, 1, 2, 0), (1, 8, 23, 23, 16, 7, 7, 2, 3), (2, 128, 7, 7, 256, 3, 3, 1, 1),
])
def test_conv_matches_oracle(oracle, geom):
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=3)
    got = _run(x, w, stride, pad)
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    assert got.shape == y32.shape
    util.assert_f16_close(got, y32, f"conv {geom}")


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
def test_conv_tile_widths(oracle, bn):
    geom = (2, 32, 10, 10, 72, 3, 3, 1, 1)
    x, w = datagen.c4_conv(*geom, seed=8)
    cfg = ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64)
    got = _run(x, w, 1, 1, cfg)
    _, y32 = oracle.conv2d_nhwc_f16(x, w, 1, 1)
    util.assert_f16_close(got, y32, f"conv bn={bn}")


def test_conv_split_k(oracle):
    geom = (1, 64, 7, 7, 64, 3, 3, 1, 1)
    x, w = datagen.c4_conv(*geom, seed=9)
    cfg = ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64, split_k=3)
    got = _run(x, w, 1, 1, cfg)
    _, y32 = oracle.conv2d_nhwc_f16(x, w, 1, 1)
    util.assert_f16_close(got, y32, "conv split-K")


def test_conv_golden_vectors_from_reference_composition():
    g = np.load(os.path.join(GOLD, "conv_ref.npz"))
    for i in range(6):
        B, C, H, W, OC, kh, kw, stride, pad = (int(v) for v in g[f"c{i}_geom"])
        x = np.ascontiguousarray(g[f"c{i}_x_nchw"].transpose(0, 2, 3, 1))
        w = np.ascontiguousarray(g[f"c{i}_w_oihw"].transpose(0, 2, 3, 1))
        Cs = ops.conv_stored_channels(C, H, W, OC, kh, kw, stride, pad)
        if Cs != C:      # the 3-channel first layer is stored with a zero fourth channel
            x = np.concatenate([x, np.zeros(x.shape[:3] + (Cs - C,), np.float16)], axis=3)
            w = np.concatenate([w, np.zeros(w.shape[:3] + (Cs - C,), np.float16)], axis=3)
        got = _run(x, w, stride, pad)
        util.assert_f16_close(got, g[f"c{i}_y_nhwc"].astype(np.float32), f"golden conv {i}")
        if (C, OC, kh, kw, stride, pad) == (64, 64, 3, 3, 1, 1):      # also through the row-pair kernel
            got = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64, conv_gather=4))
            util.assert_f16_close(got, g[f"c{i}_y_nhwc"].astype(np.float32), f"golden conv {i}, row-pair kernel")


def test_conv_delta_kernel_is_a_shift():
    """A 3x3 filter that is 1 at tap (0, 2) for channel c -> c copies the input shifted by (-1, +1)."""
    B, C, H, W = 2, 16, 12, 12
    rng = np.random.default_rng(0)
    x = rng.standard_normal((B, H, W, C)).astype(np.float16)
    w = np.zeros((C, 3, 3, C), np.float16)
    w[np.arange(C), 0, 2, np.arange(C)] = 1
    got = _run(x, w, 1, 1)
    want = np.zeros_like(x)
    want[:, 1:, :-1, :] = x[:, :-1, 1:, :]
    assert np.array_equal(got, want)


@pytest.mark.parametrize("layer", datagen.C4_LAYERS)
def test_conv_benchmark_layers_whole_output(oracle, layer):
    """Full-size ResNet-style layers at batch 32: all 32 images against the oracle, and exact
    linearity on the whole output."""
    B, C, H, W, OC, kh, kw, stride, pad = layer
    x, w = datagen.c4_conv(*layer, seed=3)
    xd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda()
    y = ops.conv2d_f16_nhwc(xd, wd, stride, pad)
    y2 = ops.conv2d_f16_nhwc(xd * 2, wd, stride, pad)
    torch.cuda.synchronize()
    ops.check_status()
    normal = y.abs() > 2.0 ** -14           # subnormal outputs sit on an absolute grid
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert (y2.float() - 2 * y.float()).abs().max().item() <= 2.0 ** -23
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    yh = y.cpu().numpy()
    util.assert_f16_close(yh, y32, f"layer {layer}")
    for img in range(B):          # no image may hide behind the norm of the others
        util.assert_f16_close(yh[img], y32[img], f"layer {layer} image {img}")


@pytest.mark.parametrize("geom", [
    (2, 64, 32, 32, 64, 3, 3, 1, 1),      # 3x3 same-size: padding on all four sides
    (3, 64, 30, 30, 72, 3, 3, 1, 1),      # M = 2700: tiles start mid-row and the last one is ragged
    (2, 128, 33, 31, 64, 3, 3, 2, 1),     # stride 2, odd sizes, two 64-channel blocks per tap
    (2, 64, 40, 40, 128, 1, 1, 2, 0),     # strided 1x1 (ResNet downsample)
    (2, 64, 31, 37, 64, 3, 3, 3, 0),      # stride 3 that does not divide the extent, no padding
    (2, 64, 24, 24, 32, 5, 5, 1, 2),      # 5x5
    (1, 64, 40, 40, 64, 7, 7, 2, 3),      # 7x7 stride 2 pad 3
    (2, 64, 32, 32, 64, 1, 3, 1, 1),      # 1x3 filter with padding also on the 1-tap axis
    (2, 192, 20, 20, 80, 3, 3, 1, 1),     # three channel blocks, narrow ragged N
])
def test_conv_im2col_tensor_map_matches_gather_and_oracle(oracle, geom):
    """Activations through the im2col tensor map (C a multiple of 64, tensor of 128 KiB or more)
    against the gathering producer on the same tile configuration -- same accumulation order, so
    the two must agree bit for bit -- and against the oracle."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    assert C % 64 == 0 and B * H * W * C * 2 >= 131072
    x, w = datagen.c4_conv(*geom, seed=21)
    bn = 64 if OC <= 64 else 128
    tma = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64))
    gather = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64, conv_gather=1))
    assert np.array_equal(tma, gather)
    auto = _run(x, w, stride, pad)
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    util.assert_f16_close(tma, y32, f"im2col conv {geom}")
    util.assert_f16_close(auto, y32, f"im2col conv {geom} default configuration")


@pytest.mark.parametrize("geom", [
    (2, 64, 32, 32, 64, 3, 3, 1, 1),      # Wp = 34, three output rows per block, 64-wide tiles
    (3, 64, 30, 30, 72, 3, 3, 1, 1),      # ragged output channels, odd number of row blocks
    (2, 128, 28, 28, 128, 3, 3, 1, 1),    # two channel blocks per tap (window ring wraps inside an item)
    (2, 64, 14, 14, 256, 3, 3, 1, 1),     # Wp = 16: eight rows per block, two output-channel tiles
    (5, 64, 7, 7, 64, 3, 3, 1, 1),        # one block per image, odd number of blocks: last item has one block
    (2, 64, 24, 24, 32, 5, 5, 1, 2),      # 5x5 window
    (2, 64, 20, 20, 64, 3, 3, 1, 0),      # no padding: Wp = W, output smaller than input
    (1, 64, 40, 40, 64, 1, 3, 1, 1),      # 1x3 filter with padding also on the 1-tap axis
    (3, 192, 20, 20, 80, 3, 3, 1, 1),     # three channel blocks
    (1, 64, 56, 56, 64, 3, 3, 1, 1),      # Wp = 58: two rows per block, 116 of 128 accumulator rows used
])
def test_conv_window_resident_kernel(oracle, geom):
    """Stride-1 convolution with the input window resident in shared memory (conv_gather = 3): every
    filter tap reads the same buffer through a shifted matrix descriptor."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=23)
    bn = 64 if OC <= 64 else 128
    got = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64, conv_gather=3))
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    assert got.shape == y32.shape
    util.assert_f16_close(got, y32, f"window-resident conv {geom}")


@pytest.mark.parametrize("geom", [
    (1, 64, 8, 8, 64, 3, 3, 1, 1),         # one item per CTA, most accumulator rows junk
    (2, 64, 56, 56, 64, 3, 3, 1, 1),       # the ResNet stage-1 layer: 116 of 128 rows live
    (3, 64, 7, 13, 64, 3, 3, 1, 1),        # odd height: the last row pair of an image has one row
    (2, 64, 33, 62, 64, 3, 3, 1, 1),       # widest row (Wp = 64): the last tap's junk rows reach past the window
    (40, 64, 56, 48, 64, 3, 3, 1, 1),      # 1120 items: seven or eight per CTA, window and accumulator rings wrap
    (300, 64, 5, 50, 64, 3, 3, 1, 1),      # three row pairs per image: strips cross images every few items
])
def test_conv_row_pair_kernel(oracle, geom):
    """3 x 3 / 1, 64 -> 64 channels with the pixels on the accumulator rows (conv_gather = 4): every tap reads the
    resident window through a shifted matrix descriptor; same summation order as the implicit GEMM, so the same bits."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=41)
    got = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64, conv_gather=4))
    other = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64))
    assert np.array_equal(got, other)
    for img in sorted({0, B - 1}):
        _, y32 = oracle.conv2d_nhwc_f16(x[img:img + 1], w, stride, pad)
        util.assert_f16_close(got[img:img + 1], y32, f"row-pair conv {geom} image {img}")
    auto = _run(x, w, stride, pad)       # the library's own choice (this kernel where its tile fits)
    assert np.allclose(auto.astype(np.float32), other.astype(np.float32), rtol=1e-2, atol=2e-3)


def test_convolutions_with_a_fixed_kernel_say_so_in_the_default_config():
    """3 x 3 / 1 at 64 -> 64 channels gets the row-pair kernel (conv_gather = 4) where its tile fits and there are a
    few row pairs per SM; the 4-channel first layer needs no workspace; everything else keeps a tunable tile."""
    import ctypes
    from helix_b200 import _lib
    from helix_b200._lib import Cfg, Launch
    lib = _lib.load()

    def default(geom, max_ctas=0):
        l = Launch()
        l.op = _lib.OP_CONV_F16
        for i, v in enumerate(geom):
            l.conv[i] = v
        l.cfg.max_ctas = max_ctas
        c = Cfg()
        assert lib.helix_default_config(ctypes.byref(l), ctypes.byref(c)) == 0
        return c, lib.helix_workspace_bytes(ctypes.byref(l))
    # (N, H, W, C, KO, R, S, stride, pad)
    c, ws = default((32, 56, 56, 64, 64, 3, 3, 1, 1))
    assert c.conv_gather == 4 and (c.tile_m, c.tile_n, c.split_k, c.stream_k, c.swap_ab) == (128, 64, 1, 0, 0) and ws == 0
    assert default((32, 56, 56, 64, 64, 3, 3, 1, 1), max_ctas=36)[0].conv_gather == 4      # one of four launch chains
    assert default((2, 56, 56, 64, 64, 3, 3, 1, 1))[0].conv_gather == 0                     # 56 row pairs on 148 SMs
    assert default((32, 28, 28, 64, 64, 3, 3, 1, 1))[0].conv_gather == 0                    # 30 of 64 pixel slots per row
    assert default((32, 56, 56, 64, 128, 3, 3, 1, 1))[0].conv_gather == 0
    assert default((32, 56, 56, 128, 64, 3, 3, 1, 1))[0].conv_gather == 0
    assert default((32, 56, 56, 64, 64, 3, 3, 2, 1))[0].conv_gather == 0
    assert default((32, 224, 224, 4, 64, 7, 7, 2, 3))[1] == 0


def test_conv_row_pair_kernel_refuses_other_geometries():
    x = torch.zeros((1, 16, 16, 128), dtype=torch.float16, device="cuda")
    w = torch.zeros((64, 3, 3, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.conv2d_f16_nhwc(x, w, 1, 1, cfg=ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64, conv_gather=4))


@pytest.mark.parametrize("geom", [
    (1, 4, 16, 16, 64, 7, 7, 2, 3),        # one item per CTA
    (2, 4, 224, 224, 64, 7, 7, 2, 3),      # the first layer of an RGB network, two images
    (4, 4, 1200, 16, 64, 7, 7, 2, 3),      # 2400 output rows: eight items per CTA, the 16-slot row ring wraps, strips cross images
    (300, 4, 20, 24, 64, 7, 7, 2, 3),      # ten output rows per image: every strip crosses images, clipped rows top and bottom
    (3, 4, 30, 50, 64, 7, 7, 2, 3),        # all four channels non-zero
    (2, 4, 64, 64, 64, 3, 3, 2, 1),        # 3 x 3: taps at window positions 1..3
    (2, 4, 64, 64, 128, 5, 5, 2, 2),       # 128 output channels: two accumulators, two staging boxes per item
    (5, 4, 40, 256, 128, 8, 6, 2, 2),      # widest row (128 output pixels), eight filter rows, even pad
    (2, 4, 33, 32, 64, 4, 2, 2, 0),        # no padding, odd height
])
def test_conv_four_channel_first_layer_kernel(oracle, geom):
    """Stride-2 convolution over 4 stored channels: the matrix descriptor reads the overlapping windows straight
    from raw image rows in shared memory (no im2col anywhere)."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=31)
    assert ops.conv_stored_channels(3, H, W, OC, kh, kw, stride, pad) == 4
    got = _run(x, w, stride, pad)
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    assert got.shape == y32.shape
    util.assert_f16_close(got, y32, f"first-layer conv {geom}")
    if kh == 7 and B == 2:
        # the same layer with the fourth channel zero and 8 stored channels goes through the gather kernel
        x[..., 3:] = 0
        x8 = np.zeros((B, H, W, 8), np.float16)
        w8 = np.zeros((OC, kh, kw, 8), np.float16)
        x8[..., :4], w8[..., :4] = x, w
        util.assert_f16_close(_run(x, w, stride, pad), oracle.conv2d_nhwc_f16(x8, w8, stride, pad)[1], "3 + 1 channels")


def test_conv_first_layer_full_batch_against_the_gather_kernel(oracle):
    """32 x 224 x 224 x 3 -> 64, 7 x 7 / 2: twelve items per CTA.  First and last image against the oracle, every
    image against the implicit-GEMM kernel on the same data stored with 8 channels (different summation order)."""
    geom = (32, 4, 224, 224, 64, 7, 7, 2, 3)
    x, w = datagen.c4_conv(*geom, seed=32)
    x[..., 3:] = 0
    w[..., 3:] = 0
    refs = {img: oracle.conv2d_nhwc_f16(x[img:img + 1], w, 2, 3)[1] for img in (0, 31)}
    for rep in range(3):   # rows are handed between warps through barriers: repeat
        got = _run(x, w, 2, 3)
        for img, y32 in refs.items():
            util.assert_f16_close(got[img:img + 1], y32, f"first layer image {img} run {rep}")
    x8 = np.zeros((32, 224, 224, 8), np.float16)
    w8 = np.zeros((64, 7, 7, 8), np.float16)
    x8[..., :4], w8[..., :4] = x, w
    other = _run(x8, w8, 2, 3)
    diff = np.abs(got.astype(np.float32) - other.astype(np.float32))
    assert float(diff.max()) <= 4e-3, float(diff.max())     # two fp16 roundings of sums of magnitude ~1


def test_conv_four_channels_outside_the_first_layer_kernel_are_refused():
    x = torch.zeros((1, 16, 16, 4), dtype=torch.float16, device="cuda")
    w = torch.zeros((64, 3, 3, 4), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception):
        ops.conv2d_f16_nhwc(x, w, 1, 1)      # stride 1: pixels must be 16 bytes
    assert ops.conv_stored_channels(3, 16, 16, 64, 3, 3, 1, 1) == 8


@pytest.mark.parametrize("geom,bn", [
    ((2, 64, 32, 32, 64, 3, 3, 1, 1), 256),     # 64 output channels on half of the 128 rows
    ((3, 64, 30, 30, 72, 3, 3, 1, 1), 256),     # ragged channels (72) and pixels (2700)
    ((2, 128, 33, 31, 128, 3, 3, 2, 1), 128),   # stride 2, two channel blocks per tap
    ((2, 64, 40, 40, 136, 1, 1, 2, 0), 256),    # two row tiles of output channels (128 + 8)
    ((1, 64, 40, 40, 64, 7, 7, 2, 3), 64),
    ((4, 192, 20, 20, 80, 3, 3, 1, 1), 256),
])
def test_conv_pixels_on_wide_axis(oracle, geom, bn):
    """swap_ab for convolutions: output channels on the 128-row axis of the tile, bn pixels per im2col box
    on the other; each warp store writes 32 consecutive channels of one pixel."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=29)
    got = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64, swap_ab=1))
    _, y32 = oracle.conv2d_nhwc_f16(x, w, stride, pad)
    assert got.shape == y32.shape
    util.assert_f16_close(got, y32, f"swapped conv {geom} bn={bn}")
    plain = _run(x, w, stride, pad, ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=64, tile_k=64))
    assert np.array_equal(got, plain)            # same K order per output element: bit-identical


@pytest.mark.parametrize("geom,bn", [((2, 64, 14, 14, 128, 3, 3, 1, 1), 128), ((5, 32, 9, 9, 72, 3, 3, 2, 1), 64),
                                     ((32, 128, 28, 28, 128, 3, 3, 1, 1), 128)])
def test_conv_stream_k(oracle, geom, bn):
    B, C, H, W, OC, kh, kw, stride, pad = geom
    x, w = datagen.c4_conv(*geom, seed=13)
    cfg = ops.make_cfg(OP_CONV_F16, tile_m=128, tile_n=bn, tile_k=64, stream_k=1)
    got = _run(x, w, stride, pad, cfg)
    sl = slice(0, min(B, 3))
    _, y32 = oracle.conv2d_nhwc_f16(x[sl], w, stride, pad)
    util.assert_f16_close(got[sl], y32, f"stream-K conv {geom}")
    if B > 3:
        _, y32 = oracle.conv2d_nhwc_f16(x[-1:], w, stride, pad)
        util.assert_f16_close(got[-1:], y32, f"stream-K conv {geom} last image")


# ----------------------------------------------------------------------------- true-fp32 convolution
@pytest.mark.parametrize("geom", [
    (2, 16, 12, 12, 24, 3, 3, 1, 1),       # 3x3 same-size
    (2, 3, 37, 41, 20, 7, 7, 2, 3),        # 3 input channels: scalar column kernel, K = 147 (unaligned GEMM path)
    (3, 32, 9, 9, 40, 1, 1, 1, 0),         # 1x1: the activations are the column matrix
    (2, 8, 15, 17, 12, 5, 5, 2, 2),        # 5x5 stride 2
    (1, 20, 10, 10, 130, 3, 3, 3, 0),      # stride 3, more output channels than one tile
    (2, 64, 14, 14, 64, 1, 1, 2, 0),       # strided 1x1 needs the column matrix
])
def test_conv_f32_matches_the_fmaf_chain(oracle, geom):
    """Column matrix + FFMA GEMM: every output is the fmaf chain over (r, s, c) ascending, bit for bit, and
    within 1e-5 of the multiply-then-add loop."""
    B, C, H, W, OC, kh, kw, stride, pad = geom
    rng = np.random.default_rng(sum(geom))
    x = rng.uniform(-1, 1, (B, H, W, C)).astype(np.float32)
    w = (rng.standard_normal((OC, kh, kw, C)) * (2.0 / (C * kh * kw)) ** 0.5).astype(np.float32)
    y = ops.conv2d_f32_nhwc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), stride, pad)
    torch.cuda.synchronize()
    ops.check_status()
    got = y.cpu().numpy()
    want = oracle.conv2d_nhwc_f32(x, w, stride, pad, fma=True)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), geom
    util.assert_f32_close(got, oracle.conv2d_nhwc_f32(x, w, stride, pad, fma=False), f"fp32 conv {geom}")


def test_conv_f32_workspace_contract():
    from helix_b200._lib import HelixError, Launch, OP_CONV_F32, load
    import ctypes
    x = torch.rand((2, 10, 10, 8), device="cuda")
    w = torch.rand((16, 3, 3, 8), device="cuda")
    y = torch.empty((2, 10, 10, 16), device="cuda")
    l = ops.launch_conv2d_f32(x, w, y, 1, 1)
    need = load().helix_workspace_bytes(ctypes.byref(l))
    M, K = 2 * 10 * 10, 3 * 3 * 8
    assert need >= (M * K + K * 16) * 4 and need % 256 == 0
    l.ws_bytes = need - 256
    with pytest.raises(HelixError) as e:
        ops.run(l)
    assert e.value.status == -3                                   # workspace missing or too small
    l1 = ops.launch_conv2d_f32(torch.rand((1, 6, 6, 8), device="cuda"), torch.rand((4, 1, 1, 8), device="cuda"),
                               torch.empty((1, 6, 6, 4), device="cuda"), 1, 0)
    assert load().helix_workspace_bytes(ctypes.byref(l1)) == 256  # 1x1: only the transposed weights (8 x 4 floats)
