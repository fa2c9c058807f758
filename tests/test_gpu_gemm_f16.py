"""GPU parity: tcgen05 fp16 GEMM (fp32 accumulate) through the C ABI vs the CPU oracle."""
import os

import numpy as np
import pytest
import torch

from helix_b200 import datagen, ops
from helix_b200._lib import OP_GEMM_F16
from tests import util

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _run(a, b_nk, cfg=None):
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b_nk).cuda()
    shape = (*a.shape[:-1], b_nk.shape[-2])
    out = torch.full(shape, float("nan"), dtype=torch.float16, device="cuda")
    ops.run(ops.launch_gemm_f16(ad, bd, out, cfg))
    torch.cuda.synchronize()
    ops.check_status()
    return out.cpu().numpy()


def _cfg(bn, split_k=1, swap=0, stages=0):
    return ops.make_cfg(OP_GEMM_F16, tile_m=128, tile_n=bn, tile_k=64, stages=stages, split_k=split_k, swap_ab=swap)


def test_single_tile_identity_known_answer():
    """One 128x128x64 tile with B = I: the output must reproduce A exactly (checks descriptors,
    swizzle, TMEM lane mapping and the epilogue addressing without any rounding)."""
    rng = np.random.default_rng(0)
    a = rng.standard_normal((128, 64)).astype(np.float16)
    b = np.zeros((128, 64), np.float16)
    b[np.arange(64), np.arange(64)] = 1
    got = _run(a, b, _cfg(128))
    assert np.array_equal(got[:, :64], a)
    assert np.all(got[:, 64:] == 0)


def test_one_hot_rows_and_k_steps():
    """Each row of A selects one k: exercises all four K=16 steps of a slab and several slabs."""
    K = 256
    a = np.zeros((128, K), np.float16)
    a[np.arange(128), (np.arange(128) * 37) % K] = 1
    rng = np.random.default_rng(1)
    b = rng.standard_normal((256, K)).astype(np.float16)
    got = _run(a, b, _cfg(256))
    want = b[:, (np.arange(128) * 37) % K].T
    assert np.array_equal(got, want)


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 512), (200, 136, 72), (1, 8, 8), (300, 1000, 264)])
def test_gemm_tiles_and_edges(oracle, shape, bn):
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=2)
    got = _run(a, b, _cfg(bn))
    _, ref32 = oracle.hgemm_naive(a, b)
    util.assert_f16_close(got, ref32, f"gemm {shape} bn={bn}")


@pytest.mark.parametrize("bn,shape", [(16, (16, 1100, 512)), (32, (24, 300, 136)), (128, (128, 512, 1024)), (64, (5, 129, 64))])
def test_gemm_swap_ab(oracle, bn, shape):
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=3)
    got = _run(a, b, _cfg(bn, swap=1))
    _, ref32 = oracle.hgemm_naive(a, b)
    util.assert_f16_close(got, ref32, f"swap gemm {shape} bn={bn}")


@pytest.mark.parametrize("split,swap", [(2, 0), (4, 0), (3, 1), (8, 1)])
def test_gemm_split_k(oracle, split, swap):
    M, N, K = (48, 400, 2048)
    a, b = datagen.c3_gemm(M, N, K, seed=4)
    cfg = _cfg(64 if swap else 128, split_k=split, swap=swap)
    got = _run(a, b, cfg)
    again = _run(a, b, cfg)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), "split-K reduction must be deterministic"
    _, ref32 = oracle.hgemm_naive(a, b)
    util.assert_f16_close(got, ref32, f"split_k={split} swap={swap}")


def test_gemm_split_k_needs_no_clean_workspace_and_replays_from_a_graph(oracle):
    """The split-K arrival counters are tagged per launch and left at zero by the CTA that completes a tile:
    a workspace full of garbage works, several tiles per CTA and ragged edges work, the slices are summed in
    slice order whoever arrives last (same bits every time), and a captured launch can be replayed."""
    M, N, K = 1000, 520, 4096          # 8 x 3 tiles of 128 x 256 (ragged), 64 K slabs cut in 5
    a, b = datagen.c3_gemm(M, N, K, seed=14)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    cfg = _cfg(256, split_k=5)
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    l = ops.launch_gemm_f16(ad, bd, out, cfg)
    ws = torch.randint(0, 255, (l.ws_bytes,), dtype=torch.uint8, device="cuda")     # garbage, counters included
    ws[:4096] = 0xFF
    l = ops.launch_gemm_f16(ad, bd, out, cfg, ws=ws)
    ops.run(l)
    torch.cuda.synchronize()
    ops.check_status()
    first = out.clone()
    _, ref32 = oracle.hgemm_fast(a, b)
    util.assert_f16_close(first.cpu().numpy(), ref32, "split-K on a dirty workspace")
    for _ in range(3):
        out.zero_()
        ops.run(l)
        torch.cuda.synchronize()
        assert torch.equal(out, first)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.run(l)
        ops.run(l)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, first)
    ops.check_status()
    # a narrow tile without the TMA store path (N not a multiple of 8) and a batch
    a2, b2 = datagen.c3_gemm(300, 100, 1024, seed=15, batch=3)
    got = _run(a2, b2, _cfg(64, split_k=4))
    for i in range(3):
        _, r = oracle.hgemm_naive(a2[i], b2[i])
        util.assert_f16_close(got[i], r, f"batched split-K entry {i}")
    a3, b3 = datagen.c3_gemm(200, 97, 1024 + 8, seed=16)
    _, r3 = oracle.hgemm_naive(a3, b3)
    util.assert_f16_close(_run(a3, b3, _cfg(32, split_k=3)), r3, "split-K, N = 97")


def test_gemm_many_tiles_persistent_and_stage_wrap(oracle):
    """More tiles than SMs and more K slabs than stages: several accumulator and ring phases."""
    M, N, K = 2048, 2304, 1024
    a, b = datagen.c3_gemm(M, N, K, seed=5)
    _, ref32 = oracle.hgemm_fast(a, b)
    for bn, stages in [(128, 0), (256, 2), (64, 3)]:
        got = _run(a, b, _cfg(bn, stages=stages))
        util.assert_f16_close(got, ref32, f"persistent bn={bn} stages={stages}")


def test_gemm_strided_batch(oracle):
    """Batched QK^T-like shape: 6 x (160, 96, 64)."""
    a, b = datagen.c3_gemm(160, 96, 64, seed=6, batch=6)
    got = _run(a, b)
    for i in range(6):
        _, ref32 = oracle.hgemm_naive(a[i], b[i])
        util.assert_f16_close(got[i], ref32, f"batch {i}")


def test_gemm_default_config_on_sweep_shapes_reduced(oracle):
    """The library's own choice (incl. swap / split-K) on scaled-down versions of the sweep shapes."""
    for (M, N, K) in [(512, 512, 512), (16, 1376, 512), (128, 512, 1376), (256, 1792, 512)]:
        a, b = datagen.c3_gemm(M, N, K, seed=2)
        got = _run(a, b)
        _, ref32 = oracle.hgemm_fast(a, b)
        util.assert_f16_close(got, ref32, f"default {M}x{N}x{K}")


def test_gemm_golden_vectors_from_reference_loop():
    g = np.load(os.path.join(GOLD, "hgemm_ref.npz"))
    for n in sorted({k.split("_a")[0] for k in g.files if k.endswith("_a")}):
        a, b_kn = g[n + "_a"], g[n + "_b_kn"]
        if a.shape[1] % 8:
            continue  # leading dimension rule (16 bytes); odd K goes through the padded host entry point
        got = _run(a, np.ascontiguousarray(b_kn.T))
        util.assert_f16_close(got, g[n + "_c"].astype(np.float32), n)


def test_gemm_host_entry_point_pads_odd_k(oracle, lib):
    import ctypes
    g = np.load(os.path.join(GOLD, "hgemm_ref.npz"))
    a, b_kn = g["h1_a"], g["h1_b_kn"]           # K = 129
    b_nk = np.ascontiguousarray(b_kn.T)
    c = np.empty((a.shape[0], b_nk.shape[0]), np.float16)
    rc = lib.helix_gemm_f16_host(a.ctypes.data_as(ctypes.c_void_p), b_nk.ctypes.data_as(ctypes.c_void_p),
                                 c.ctypes.data_as(ctypes.c_void_p), a.shape[0], b_nk.shape[0], a.shape[1])
    assert rc == 0
    util.assert_f16_close(c, g["h1_c"].astype(np.float32), "host entry, K=129")


def test_gemm_rejects_misaligned_leading_dimension():
    a = torch.zeros((16, 20), dtype=torch.float16, device="cuda")
    b = torch.zeros((16, 20), dtype=torch.float16, device="cuda")
    with pytest.raises(Exception) as e:
        ops.gemm_f16(a, b)
    assert "-2" in str(e.value)


@pytest.mark.parametrize("shape", datagen.C3_SHAPES)
def test_gemm_full_size_against_the_oracle_and_exact_properties(oracle, shape):
    """The five benchmark shapes at full size.  The whole output is compared with the oracle's blocked fp16
    GEMM (fp32 partial sums; seconds on a multi-core host even at 8192^3).  Two exact, size-independent
    properties ride along: rows of A that are one-hot must reproduce columns of B exactly, and scaling A by 2
    (exact in fp16) must scale C by exactly 2 wherever C is a normal fp16 number (subnormal outputs sit on
    an absolute grid, so there 2*round(c) may differ from round(2c) by one grid step)."""
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=2)
    sel = (np.arange(M) * 7919) % K
    a[::5] = 0
    a[np.arange(0, M, 5), sel[::5]] = 1
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c1 = ops.gemm_f16(ad, bd)
    c2 = ops.gemm_f16(ad * 2, bd)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(c1[::5], bd[:, torch.from_numpy(sel[::5]).cuda()].t().contiguous())
    normal = c1.abs() > 2.0 ** -14
    assert torch.equal(c2[normal], (c1 * 2)[normal])
    assert (c2.float() - 2 * c1.float()).abs().max().item() <= 2.0 ** -23
    del c2, normal
    _, ref32 = oracle.hgemm_fast(a, b)
    util.assert_f16_close(c1.cpu().numpy(), ref32, f"full-size {shape}")


def _sk(bn, swap=0):
    return ops.make_cfg(OP_GEMM_F16, tile_m=128, tile_n=bn, tile_k=64, swap_ab=swap, stream_k=1, load_group=2)


@pytest.mark.parametrize("bn,swap,shape", [
    (128, 0, (256, 384, 2048)),      # 6 tiles < SMs: every tile is shared by many CTAs
    (64, 0, (1000, 520, 1096)),      # ragged edges, K tail
    (16, 1, (16, 1100, 1024)),       # skinny M, swapped
    (256, 0, (2560, 2304, 512)),     # 180 tiles: one whole wave + a dealt-out tail
    (128, 0, (2048, 2304, 320)),     # 288 tiles, 5 slabs each: tail tiles touched by two CTAs
    (32, 1, (24, 4000, 200)),
    (128, 0, (128, 128, 64)),        # one tile, one slab
])
def test_gemm_stream_k(oracle, bn, swap, shape):
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=11)
    cfg = _sk(bn, swap)
    got = _run(a, b, cfg)
    again = _run(a, b, cfg)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16)), "stream-K fix-up must be deterministic"
    _, ref32 = oracle.hgemm_fast(a, b)
    util.assert_f16_close(got, ref32, f"stream-K {shape} bn={bn} swap={swap}")


def test_gemm_stream_k_batched(oracle):
    a, b = datagen.c3_gemm(200, 136, 192, seed=12, batch=5)
    got = _run(a, b, _sk(64))
    for i in range(5):
        _, ref32 = oracle.hgemm_naive(a[i], b[i])
        util.assert_f16_close(got[i], ref32, f"stream-K batch {i}")


def test_gemm_stream_k_needs_workspace():
    a = torch.zeros((256, 256), dtype=torch.float16, device="cuda")
    b = torch.zeros((384, 256), dtype=torch.float16, device="cuda")
    out = torch.zeros((256, 384), dtype=torch.float16, device="cuda")
    l = ops.launch_gemm_f16(a, b, out, _sk(128))
    assert l.ws_bytes > 0
    l.ws, l.ws_bytes = None, 0
    with pytest.raises(Exception) as e:
        ops.run(l)
    assert "-3" in str(e.value)


def _pair(bn, stages=0):
    return ops.make_cfg(OP_GEMM_F16, tile_m=128, tile_n=bn, tile_k=64, stages=stages, cta_group=2)


@pytest.mark.parametrize("bn,shape", [
    (256, (256, 256, 64)),        # one pair tile, one slab
    (128, (256, 128, 256)),
    (256, (512, 768, 1024)),      # several tiles per pair, ring wraps
    (256, (300, 520, 264)),       # ragged M, N, K
    (128, (2048, 2304, 512)),     # more tiles than CTA pairs
    (256, (100, 40, 72)),         # smaller than one tile
    (192, (256, 192, 128)),       # 96-row B halves, three 64-column epilogue chunks
    (192, (1024, 1000, 520)),     # ragged last 192-wide column of tiles, ring wraps
    (192, (2304, 2112, 256)),     # more tiles than CTA pairs
])
def test_gemm_cta_pairs(oracle, bn, shape):
    """tcgen05.mma.cta_group::2: two CTAs share a 256 x BN tile."""
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=14)
    got = _run(a, b, _pair(bn))
    _, ref32 = oracle.hgemm_fast(a, b)
    util.assert_f16_close(got, ref32, f"CTA pairs {shape} bn={bn}")


@pytest.mark.parametrize("bn,shape", [
    (256, (1024, 768, 512)),      # 12 tiles on 74 pairs: every tile is shared by two pairs
    (256, (256, 1280, 832)),      # 13 slabs per tile, ranges of 4: ranges straddle two tiles
    (192, (2304, 2112, 256)),     # one whole round plus dealt-out tiles that each stay with one pair
    (256, (2560, 2048, 1024)),    # 80 tiles: one round, six tiles dealt out over all pairs
    (128, (300, 520, 264)),       # ragged M, N, K
])
def test_gemm_cta_pairs_stream_k(oracle, bn, shape):
    """CTA pairs with the K slabs of the last partial round dealt to all pairs (fp32 slots + fix-up)."""
    M, N, K = shape
    a, b = datagen.c3_gemm(M, N, K, seed=17)
    cfg = ops.make_cfg(OP_GEMM_F16, tile_m=128, tile_n=bn, tile_k=64, cta_group=2, stream_k=1)
    got = _run(a, b, cfg)
    _, ref32 = oracle.hgemm_fast(a, b)
    util.assert_f16_close(got, ref32, f"CTA pairs stream-K {shape} bn={bn}")
    again = _run(a, b, cfg)
    assert np.array_equal(got, again)            # fixed summation order: bit-reproducible


def test_gemm_cta_pairs_known_answer_and_batch(oracle):
    K = 128
    a = np.zeros((256, K), np.float16)
    a[np.arange(256), (np.arange(256) * 5) % K] = 1
    b = np.random.default_rng(3).standard_normal((256, K)).astype(np.float16)
    got = _run(a, b, _pair(256))
    assert np.array_equal(got, b[:, (np.arange(256) * 5) % K].T)   # rows 128..255 come from the odd CTA
    ab, bb = datagen.c3_gemm(260, 136, 192, seed=15, batch=3)
    gb = _run(ab, bb, _pair(128, stages=2))
    for i in range(3):
        _, ref32 = oracle.hgemm_naive(ab[i], bb[i])
        util.assert_f16_close(gb[i], ref32, f"CTA pairs batch {i}")


def test_gemm_independent_launch_chain_matches_ordered(oracle):
    """HELIX_LAUNCH_INDEPENDENT lets consecutive launches overlap at their edges; results are unchanged."""
    a, b = datagen.c3_gemm(1024, 768, 512, seed=16)
    ad, bd = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    ref = ops.gemm_f16(ad, bd)
    outs = [torch.full((1024, 768), float("nan"), dtype=torch.float16, device="cuda") for _ in range(8)]
    for i, o in enumerate(outs):
        cfg = _pair(256) if i % 2 else _cfg(128)
        l = ops.launch_gemm_f16(ad, bd, o, cfg)
        l.flags = 1
        ops.run(l)
    torch.cuda.synchronize()
    ops.check_status()
    _, ref32 = oracle.hgemm_fast(a, b)
    for o in outs:
        util.assert_f16_close(o.cpu().numpy(), ref32, "independent chain")
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[3])


def test_an_independent_launch_does_not_break_the_order_of_its_neighbours(oracle):
    """A (long) -> B (short, flagged HELIX_LAUNCH_INDEPENDENT, unrelated buffers) -> C (ordered, reads A's
    output).  B does not wait for A before it works, but it waits before it exits, so C -- which waits for B --
    never starts reading A's output while A still writes it."""
    from helix_b200._lib import LAUNCH_INDEPENDENT
    a1, b1 = datagen.c3_gemm(256, 512, 8192, seed=31)          # A: 2 x 2 tiles, 128 K slabs each
    _, b2 = datagen.c3_gemm(8, 384, 512, seed=32)
    a3, b3 = datagen.c3_gemm(128, 128, 64, seed=33)            # B: one tile, one slab
    d = [torch.from_numpy(x).cuda() for x in (a1, b1, b2, a3, b3)]
    c1 = torch.zeros((256, 512), dtype=torch.float16, device="cuda")
    c2 = torch.zeros((256, 384), dtype=torch.float16, device="cuda")
    c3 = torch.zeros((128, 128), dtype=torch.float16, device="cuda")
    la = ops.launch_gemm_f16(d[0], d[1], c1, _cfg(256))
    lc = ops.launch_gemm_f16(c1, d[2], c2, _cfg(128))
    lb = ops.launch_gemm_f16(d[3], d[4], c3, _cfg(128))
    lb.flags = LAUNCH_INDEPENDENT
    ops.run(la)
    torch.cuda.synchronize()
    ops.run(lc)
    torch.cuda.synchronize()
    want = c2.clone()                                          # the chain with a host synchronisation in between
    _, ref1 = oracle.hgemm_naive(a1, b1)
    util.assert_f16_close(c1.cpu().numpy(), ref1, "first product")
    _, ref2 = oracle.hgemm_naive(c1.cpu().numpy(), b2)
    util.assert_f16_close(want.cpu().numpy(), ref2, "second product")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.run(la)
        ops.run(lb)
        ops.run(lc)
    for trial in range(20):
        c1.zero_()
        c2.zero_()
        torch.cuda.synchronize()
        if trial % 2:
            g.replay()
        else:
            ops.run(la)
            ops.run(lb)
            ops.run(lc)
        torch.cuda.synchronize()
        assert torch.equal(c2, want), trial
    ops.check_status()


@pytest.mark.parametrize("shape,bn", [((300, 200, 520), 64), ((1024, 768, 2048), 128), ((512, 1024, 4096), 256)])
def test_two_issuing_warps_give_the_same_bits(shape, bn):
    """probe bit 7: two warps issue the MMAs of alternate K slabs, their order fixed by a token that travels through
    two named barriers; the accumulation order, hence every bit of the result, is that of the single issuer."""
    M, N, K = shape
    a = torch.randn((M, K), device="cuda", dtype=torch.float16) / K ** 0.5
    b = torch.randn((N, K), device="cuda", dtype=torch.float16) / K ** 0.5
    one = ops.gemm_f16(a, b, cfg=ops.make_cfg(OP_GEMM_F16, 128, bn, 64))
    two = ops.gemm_f16(a, b, cfg=ops.make_cfg(OP_GEMM_F16, 128, bn, 64, probe=0x80))
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(one, two)
    ref = a.float() @ b.float().T
    assert float((two.float() - ref).norm() / ref.norm()) < 2e-3
    # the pair kernel: two issuing warps are its default, probe bit 9 selects the single issuer
    pair_two = ops.gemm_f16(a, b, cfg=ops.make_cfg(OP_GEMM_F16, 256, max(bn, 128), 64, cta_group=2))
    pair_one = ops.gemm_f16(a, b, cfg=ops.make_cfg(OP_GEMM_F16, 256, max(bn, 128), 64, cta_group=2, probe=0x200))
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(pair_one, pair_two)
    assert float((pair_two.float() - ref).norm() / ref.norm()) < 2e-3
