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


def test_two_lanes_match_the_serial_sweep():
    units = _reduced_units()
    serial = sweep.Sweep(units, seed=7, lanes=1)
    lanes = sweep.Sweep(units, seed=7, lanes=2)
    assert all(l.cfg.max_ctas == (ops.device_info().sm_count // 2) & ~1 for l in lanes.launches)
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
