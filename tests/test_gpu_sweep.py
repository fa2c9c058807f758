"""GPU tests of the sweep drivers: concurrent launch chains (lanes) give the results of the serial sweep."""
import pytest
import torch

from helix_b200 import ops, sweep, workloads

pytestmark = pytest.mark.gpu


def _reduced_units():
    """A few units of every kind of the model-level sweep at reduced batch (same per-row geometry)."""
    units = workloads.model_level_sweep(bert_batch=2, seq=256, resnet_batch=2)
    picked, seen = [], set()
    for u in units:
        key = (u["kind"], tuple(u["shape"]))
        if key not in seen:
            seen.add(key)
            picked.append(u)
    return picked


@pytest.mark.parametrize("nlanes", [2, 4])
def test_lanes_match_the_serial_sweep(nlanes):
    units = _reduced_units()
    serial = sweep.Sweep(units, seed=7, lanes=1)
    lanes = sweep.Sweep(units, seed=7, lanes=nlanes)
    share = lanes.lane_sms()
    sms = ops.device_info().sm_count
    assert len(share) == nlanes and all(v % 2 == 0 for v in share) and sms - 1 <= sum(share) <= sms
    assert all(l.cfg.max_ctas == share[lane] for l, lane in zip(lanes.launches, lanes.lane_of))
    n1 = serial.step()
    n2 = lanes.step()
    torch.cuda.synchronize()
    ops.check_status()
    assert n1 >= len(units) and n2 >= len(units)
    for u, (a1, b1, o1), (a2, b2, o2) in zip(units, serial.tensors, lanes.tensors):
        assert torch.equal(a1, a2) and torch.equal(b1, b2)           # same seeded operands
        # a launch limited to half the SMs may pick another tile shape; every output element is still
        # one fp32 sum over k in ascending order unless K is split, so the halves agree to rounding
        assert torch.allclose(o1.float(), o2.float(), rtol=1e-2, atol=2e-3), u


def test_lanes_inside_a_cuda_graph_replay():
    units = _reduced_units()[:12]
    sw = sweep.Sweep(units, seed=9, lanes=2)
    sw.step()
    torch.cuda.synchronize()
    want = [o.clone() for _, _, o in sw.tensors]
    for _, _, o in sw.tensors:
        o.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sw.step()
    g.replay()
    torch.cuda.synchronize()
    ops.check_status()
    for w, (_, _, o) in zip(want, sw.tensors):
        assert torch.equal(w, o)


def test_gemm_split_along_n_matches_the_unsplit_product_and_the_oracle(oracle):
    """Each rank's column slab (ranks emulated one after another on this GPU) equals the same columns of the
    one-GPU product, and sampled rows agree with the CPU oracle."""
    import numpy as np
    from helix_b200 import nsplit
    from tests.util import assert_f16_close
    M, N, K = 384, 2816, 512
    cfg = ops.make_cfg(0, tile_n=128)                  # same tile on every rank: identical summation per element
    whole = nsplit.NSplitGemm(M, N, K, seed=11, world=1, rank=0, cfg=cfg)
    whole.step()
    torch.cuda.synchronize()
    full = whole.gather()
    for world in (2, 3):
        slabs, bounds = [], []
        for r in range(world):
            g = nsplit.NSplitGemm(M, N, K, seed=11, world=world, rank=r, cfg=cfg)
            assert torch.equal(g.a, whole.a) and torch.equal(g.b, whole.b[g.n0:g.n1])
            g.step()
            torch.cuda.synchronize()
            slabs.append(g.c.cpu().numpy())
            bounds.append((g.n0, g.n1))
        ops.check_status()
        assert np.array_equal(nsplit.assemble(slabs, bounds, M, N), full)
    a = whole.a.cpu().numpy()
    b = whole.b.cpu().numpy()
    rows = [0, 127, 128, 383]
    _, ref = oracle.hgemm_naive(np.ascontiguousarray(a[rows]), b)
    assert_f16_close(full[rows], ref, "N-split GEMM")


def _check_unit_against_oracle(oracle, u, a, b, out, what):
    """One unit of the sweep against the CPU oracle: whole output for a plain GEMM, three batch entries of a
    batched GEMM, first / middle / last image of a convolution."""
    import numpy as np
    from tests.util import assert_f16_close
    s = u["shape"]
    if u["kind"] == "gemm" and len(s) == 3:
        _, ref32 = oracle.hgemm_fast(a.cpu().numpy(), b.cpu().numpy())
        assert_f16_close(out.cpu().numpy(), ref32, what)
        return 1
    if u["kind"] == "gemm":
        batch = s[3]
        for i in sorted({0, batch // 2, batch - 1}):
            _, ref32 = oracle.hgemm_naive(a[i].cpu().numpy(), b[i].cpu().numpy())
            assert_f16_close(out[i].cpu().numpy(), ref32, f"{what} batch entry {i}")
        return 1
    stride, pad = s[7], s[8]
    w = b.cpu().numpy()
    for img in sorted({0, s[0] // 2, s[0] - 1}):
        _, y32 = oracle.conv2d_nhwc_f16(np.ascontiguousarray(a[img:img + 1].cpu().numpy()), w, stride, pad)
        assert_f16_close(out[img:img + 1].cpu().numpy(), y32, f"{what} image {img}")
    return 1


@pytest.mark.parametrize("lanes", [4, 2, 1])
def test_model_level_sweep_at_full_size_against_the_oracle(oracle, lanes):
    """The benchmark's own workload and launch configuration: every GEMM of BERT-base at batch 16 / seq 512 and
    the 53 ResNet-50 convolutions at batch 32, dealt to `lanes` concurrent chains with each launch limited to
    1 / lanes of the SMs (the library re-chooses its tile for the smaller machine), independent-launch flag set.
    Every distinct shape (4 linear GEMMs, the two batched attention GEMMs, 23 convolutions, among them the 7x7
    first layer with 3 channels stored as 4, the 7x7-pixel layers and the strided 1x1 projections) is compared with
    the oracle; then the same step replayed from a CUDA graph, as the benchmark times it, must reproduce the
    eager outputs bit for bit."""
    units = workloads.model_level_sweep()
    sw = sweep.Sweep(units, seed=4000, lanes=lanes)
    n = sw.step()
    torch.cuda.synchronize()
    ops.check_status()
    assert n >= len(units)
    seen, checked = set(), 0
    for u, (a, b, out) in zip(units, sw.tensors):
        key = (u["kind"], tuple(u["shape"]))
        if key in seen:
            continue
        seen.add(key)
        checked += _check_unit_against_oracle(oracle, u, a, b, out, f"{u['name']} {u['shape']} lanes={lanes}")
    assert checked == 4 + 2 + 23
    # every unit, repeated layers included: a repeated shape must give what its first instance gave on its own data
    eager = [out.clone() for _, _, out in sw.tensors]
    for _, _, out in sw.tensors:
        out.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        sw.step()
    g.replay()
    torch.cuda.synchronize()
    ops.check_status()
    for u, want, (_, _, out) in zip(units, eager, sw.tensors):
        assert torch.equal(want, out), u["name"]
    # last instance of each repeated shape (other buffers, other position in the chains) against the oracle too
    last = {}
    for i, u in enumerate(units):
        last[(u["kind"], tuple(u["shape"]))] = i
    for key, i in last.items():
        u = units[i]
        if u["kind"] == "gemm" and i >= 6:       # a later BERT layer
            a, b, out = sw.tensors[i]
            _check_unit_against_oracle(oracle, u, a, b, out, f"{u['name']} (last instance) lanes={lanes}")
