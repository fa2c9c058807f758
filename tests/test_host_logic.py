"""CPU-only tests of the host side: cost model, shape suites, drop-in scripts, sharding, rank aggregation."""
import importlib
import json
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = os.path.join(ROOT, "helix_b200", "scripts")

from helix_b200 import costmodel, shard, workloads  # noqa: E402


def synthetic_dict():
    d = {("sm_count",): 148, ("dram_gbs_per_sm",): 40.0, ("hbm_gbs",): 6000.0}
    slab = {256: 0.45e-6, 128: 0.31e-6, 64: 0.27e-6, 32: 0.26e-6, 16: 0.25e-6}
    for key in costmodel.gemm_keys():
        d[key] = (4e-6, {256: 0.41e-6, 192: 0.33e-6}[key[2]] if key[3] == 2 else slab[key[2]])
    for bn in (256, 128, 64):
        d[("streamk_overhead", bn)] = 8e-6 + bn * 4e-8
        d[("conv_slab", bn)] = 0.6e-6
    for key in costmodel.gemv_keys():
        d[key] = (0.3e-6 + 2e-6 * (key[5] > 1), 1.0 / 6.2e12)   # as profiled: chains of independent GEMVs overlap
    return d


def test_dictionary_round_trip_is_a_python_literal(tmp_path):
    d = synthetic_dict()
    p = tmp_path / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict"
    costmodel.save(d, str(p))
    text = p.read_text()
    assert "\n" not in text.strip()
    assert eval(text) == d            # the reference loads the file with eval(lines[0])
    assert costmodel.load(str(p)) == d


def test_cost_model_picks_sensible_configurations():
    d = synthetic_dict()
    big = costmodel.cost_model(d, 8192, 8192, 8192)
    assert big[0] != 0 and big[2] == 256 and big[4] == 0
    gemv = costmodel.cost_model(d, 1, 4096, 4096)
    assert gemv[0] == 0                                   # first element 0 <=> GEMV, as in the reference's keys
    tall = costmodel.cost_model(d, 7680, 2, 2560)         # N <= 8: GEMV with the matrix on M
    assert tall[0] == 0
    skinny = costmodel.cost_model(d, 16, 11008, 4096)
    assert skinny[0] != 0 and skinny[4] == 1              # M = 16 goes on the UMMA N axis
    conv = costmodel.cost_model(d, 25088, 128, 1152, conv=True)
    assert conv[0] != 0 and conv[4] == 0                  # no swap for the gathering producer
    # unlike the reference's model, K matters: a deep K amortises the stream-K fix-up on a ragged tile count
    assert costmodel.cost_model(d, 2048, 14336, 256)[5] == 0
    assert costmodel.cost_model(d, 128, 4096, 11008)[5] == 1


def test_cost_model_wave_quantisation_uses_device_sm_count():
    d = synthetic_dict()
    key = (4, 128, 256, 1, 0, 0)
    t148 = costmodel.gemm_time(d, key, 128 * 148, 256, 4096)
    t149 = costmodel.gemm_time(d, key, 128 * 149, 256, 4096)      # one tile more than a wave
    assert t149 > 1.8 * t148 - 4e-6
    d[("sm_count",)] = 160
    assert costmodel.gemm_time(d, key, 128 * 149, 256, 4096) == pytest.approx(t148, rel=0.05)


def test_sgemm_cost_model():
    d = {("sm_count",): 148}
    for key in costmodel.sgemm_keys():
        d[key] = 1e-7 * key[0] * key[1] / (64 * 64) * (1.2 if key[0] < 128 else 1.0)
    assert costmodel.sgemm_cost_model(d, 4096, 4096, 4096)[:2] == (128, 128)
    small = costmodel.sgemm_cost_model(d, 256, 256, 1024)
    assert small[0] * small[1] < 128 * 128                       # few tiles: smaller tiles fill more SMs


def test_workloads_match_the_published_totals():
    units = workloads.model_level_sweep()
    assert len(units) == 125 and sum(u["kind"] == "conv" for u in units) == 53
    gemm = sum(workloads.unit_flops(u) for u in units if u["kind"] == "gemm")
    conv = sum(workloads.unit_flops(u) for u in units if u["kind"] == "conv")
    assert gemm == pytest.approx(1546.19e9, rel=1e-4) and conv == pytest.approx(261.58e9, rel=1e-4)
    assert len({u["shape"] for u in units if u["kind"] == "conv"}) == 23
    assert sum(workloads.unit_bytes(u) for u in units if u["kind"] == "conv") == pytest.approx(1440.6e6, rel=1e-3)


def test_lpt_partition_balances_and_is_deterministic():
    costs = [float(workloads.unit_flops(u)) for u in workloads.model_level_sweep()]
    for parts in (1, 2, 4, 8):
        p = workloads.lpt_partition(costs, parts)
        assert sorted(i for lst in p for i in lst) == list(range(len(costs)))
        loads = [sum(costs[i] for i in lst) for lst in p]
        assert max(loads) <= sum(costs) / parts + max(costs)
        assert p == workloads.lpt_partition(costs, parts)


def _digest(lists):
    import hashlib
    return hashlib.sha256(repr([[tuple(t) for t in lst] for lst in lists]).encode()).hexdigest()


def test_shape_suites_equal_the_references():
    """Counts and content hashes of the four shape-list functions, pinned from the reference's
    scripts/utils/get_benchmark_shape_list.py (the hashes are printed by make_shape_tables.py)."""
    sys.path.insert(0, SCRIPTS)
    try:
        m = importlib.import_module("utils.get_benchmark_shape_list")
    finally:
        sys.path.remove(SCRIPTS)
    gemm = m.get_gemm_op_MNKList()
    assert len(gemm) == 1274 and all(len(s) == 3 for s in gemm)
    assert _digest([gemm]) == "2f6ffeee2629219496dbe5448fd1e1cc2c29e8d6a541b58d9fa5d254c01dd6a6"
    assert (512, 1, 500000) in gemm and (1889542, 16, 66) in gemm and (2708, 16, 1433) in gemm
    llm = m.get_llm_opset_MNKList()
    assert tuple(len(x) for x in llm) == (4380, 240, 5760)
    assert _digest(llm) == "e37b93b87aac8b0f761df084fc4dcf4e742e3bded464fc27ebf1c1faba9c0d7a"
    conv = m.get_conv_op_shape_list()
    assert len(conv) == 1756 and all(len(s) == 9 for s in conv)
    assert _digest([conv]) == "dd481163f4c5c2ba0c9bef19b3378683ad84af8ed7dc36d57003bb789266cf92"
    assert (1, 1, 161, 700, 32, 5, 20, 2, 0) in conv
    cnn = m.get_cnn_opset_shape_List()
    assert tuple(len(x) for x in cnn) == (85, 340, 952)
    assert _digest(cnn) == "d012f022a264451e930529cd8dd28deef1ad1c9edb5500b3a51c6f0a50cbe9f2"


@pytest.mark.parametrize("script,args,expect", [
    ("benchmark_op_level_eval.py", ["-o", "GEMM", "-b", "x86_CPU", "-s", "Helix"], "GEMM x86_CPU Helix is not supported"),
    ("benchmark_model_level_eval.py", ["-m", "CNN", "-b", "ARM_CPU", "-s", "acl"], "CNN ARM_CPU acl is not supported"),
    ("runtime_cost.py", ["-b", "x86_CPU"], "covers the GPU backends only"),
])
def test_cli_flags_and_dispatch_without_a_gpu(script, args, expect):
    env = dict(os.environ, PYTHONPATH=SCRIPTS)
    out = subprocess.run([sys.executable, os.path.join(SCRIPTS, script)] + args, capture_output=True, text=True,
                         env=env, cwd=ROOT, timeout=120)
    assert out.returncode == 0, out.stderr
    assert expect in out.stdout


def test_backend_modules_import_lazily_and_expose_the_reference_names():
    sys.path.insert(0, SCRIPTS)
    try:
        for mod, names in [
            ("Ampere_FP16.build_Ampere_FP16", ["build_Helix_Ampere_FP16_gemm_kernel", "build_cublas_FP16_gemm_kernel",
                                               "build_cudnn_FP16_conv_kernel", "is_valid_config", "compile_kernel"]),
            ("Ampere_FP16.profile_Ampere_FP16", ["profile_Helix_Ampere_FP16_gemm_kernel"]),
            ("Ampere_FP16.changed_profile_Ampere_FP16", ["profile_Helix_Ampere_FP16_gemm_kernel"]),
            ("Ampere_FP16.Ampere_FP16_gemm", ["cost_model", "get_Ampere_FP16_gemm_Helix_result", "get_Ampere_FP16_gemm_cublas_result"]),
            ("Ampere_FP16.Ampere_FP16_conv", ["cost_model", "get_Ampere_FP16_conv_Helix_result", "get_Ampere_FP16_conv_cudnn_result"]),
            ("Ampere_FP16.Ampere_FP16_runtime_cost", ["Ampere_FP16_runtime_cost", "get_Helix_runtime_cost"]),
            ("Ampere_FP16.benchmark_Ampere_FP16_gemm", ["Ampere_FP16_Helix_op_level_GEMM_benchmark"]),
            ("Ampere_FP16.benchmark_Ampere_FP16_conv", ["Ampere_FP16_Helix_op_level_Conv_benchmark"]),
            ("Ampere_FP16.benchmark_Ampere_FP16_model_level_LLM", ["Ampere_FP16_Helix_model_level_LLM_benchmark"]),
            ("Ampere_FP16.benchmark_Ampere_FP16_model_level_CNN", ["Ampere_FP16_Helix_model_level_CNN_benchmark"]),
            ("Ampere_FP32.build_Ampere_FP32", ["build_Helix_Ampere_FP32_gemm_kernel", "build_cublas_FP32_gemm_kernel",
                                               "build_cudnn_FP32_conv_kernel", "get_copy_value"]),
            ("Ampere_FP32.profile_Ampere_FP32", ["profile_Helix_Ampere_FP32_gemm_kernel"]),
            ("Ampere_FP32.Ampere_FP32_gemm", ["cost_model", "get_Ampere_FP32_gemm_Helix_result"]),
            ("Ampere_FP32.Ampere_FP32_conv", ["cost_model", "get_Ampere_FP32_conv_Helix_result"]),
            ("Ampere_FP32.Ampere_FP32_runtime_cost", ["Ampere_FP32_runtime_cost"]),
            ("Ampere_FP32.benchmark_Ampere_FP32_model_level_CNN", ["Ampere_FP32_Helix_model_level_CNN_benchmark"]),
        ]:
            m = importlib.import_module(mod)
            for n in names:
                assert callable(getattr(m, n)), (mod, n)
        cm = importlib.import_module("Ampere_FP16.Ampere_FP16_gemm").cost_model
        assert cm(synthetic_dict(), 4096, 4096, 4096)[2] == 256
    finally:
        sys.path.remove(SCRIPTS)


# ----------------------------------------------------------------------------- sharded sweep with a fake device
def fake_device(device, unit, scale):
    time.sleep(unit["cost"] * scale)
    return {"shape": unit["name"], "ms": unit["cost"] * 1e3}


_seen = {"n": 0}


def dying_device(device, unit, scale):
    _seen["n"] += 1                        # per worker process (forked), so this counts its own units
    if device == 1 and _seen["n"] == 3:
        os._exit(17)                       # a worker that exits mid-sweep, between units
    return fake_device(device, unit, scale)


def test_sharded_sweep_two_workers_resume_and_requeue(tmp_path):
    units = [{"name": f"u{i}", "cost": 0.01 * (1 + i % 4)} for i in range(12)]
    costs = [u["cost"] for u in units]
    journal = str(tmp_path / "sweep.jsonl")
    rows, stats = shard.run_sharded(units, fake_device, [0, 1], costs, journal, fn_args=(1.0,), start_method="fork")
    assert sorted(rows) == list(range(12)) and stats["unfinished"] == 0 and not stats["failed_workers"]
    assert {r["device"] for r in rows.values()} == {0, 1}
    assert len(open(journal).read().splitlines()) == 12
    # resume: nothing left to do, no worker work repeated
    rows2, stats2 = shard.run_sharded(units, fake_device, [0, 1], costs, journal, fn_args=(1.0,), start_method="fork")
    assert stats2["resumed"] == 12 and stats2["rounds"] == 0 and sorted(rows2) == list(range(12))
    # a worker dies on the host between units: the survivor finishes its share
    journal2 = str(tmp_path / "sweep2.jsonl")
    rows3, stats3 = shard.run_sharded(units, dying_device, [0, 1], costs, journal2, fn_args=(0.1,), start_method="fork")
    assert sorted(rows3) == list(range(12)) and stats3["failed_workers"] == [1] and stats3["rounds"] == 2
    # a torn last line (killed mid-write) is ignored on resume
    with open(journal2, "a") as f:
        f.write('{"index": 99, "dev')
    assert sorted(shard.read_journal(journal2)) == list(range(12))


# ----------------------------------------------------------------------------- rank aggregation over gloo
WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import torch.distributed as dist
from helix_b200 import dist_util
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank = dist.get_rank()
dist_util.barrier(dist)
slowest = dist_util.max_over_ranks(1.0 + rank, dist)
tput = dist_util.aggregate_throughput(10.0, 1.0 + rank, dist)
total = dist_util.sum_over_ranks(3.0 + rank, dist)
each = dist_util.gather_floats(5.0 * (rank + 1), dist)
# the benchmark's partition of a fixed work list: every unit lands on exactly one rank
import importlib.util
spec = importlib.util.spec_from_file_location("bench", os.path.join({root!r}, "bench.py"))
bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)
from helix_b200 import workloads
units = bench.work_list()
parts = workloads.lpt_partition([bench.unit_estimate(u) for u in units], 2)
mine = sum(bench.unit_estimate(units[i]) for i in parts[rank])
loads = dist_util.gather_floats(mine, dist)
covered = dist_util.sum_over_ranks(len(parts[rank]), dist)
print(f"{{rank}} {{slowest}} {{tput}} {{total}} {{each[0]}} {{each[1]}} {{covered}} {{len(units)}} {{loads[0]}} {{loads[1]}}")
dist.destroy_process_group()
"""


def test_max_over_ranks_and_aggregate_throughput_world_size_2(tmp_path):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "w.py"
    script.write_text(WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, text=True) for r in (0, 1)]
    outs = [p.communicate(timeout=120)[0].split() for p in procs]
    assert all(p.returncode == 0 for p in procs)
    for rank, (r, slowest, tput, total, e0, e1, covered, n_units, l0, l1) in enumerate(outs):
        assert int(r) == rank and float(slowest) == 2.0 and float(tput) == pytest.approx(10.0)   # 2 x 10 units / 2 s
        assert float(total) == 7.0 and (float(e0), float(e1)) == (5.0, 10.0)
        assert float(covered) == float(n_units) == 1000.0
        assert abs(float(l0) - float(l1)) <= 0.01 * float(l0)        # LPT leaves the two ranks within 1 %


# ----------------------------------------------------------------------------- one GEMM split along N
def test_nsplit_slabs_tile_n_and_rows_do_not_depend_on_the_split():
    import numpy as np
    from helix_b200 import nsplit
    for N in (0, 1, 255, 256, 1000, 4096, 11008, 65536):
        for world in (1, 2, 3, 4, 8):
            bounds = [nsplit.slab_bounds(N, world, r) for r in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == N
            for (a0, a1), (b0, b1) in zip(bounds, bounds[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(n0 % nsplit.ROW_BLOCK == 0 for n0, _ in bounds)
            widths = [n1 - n0 for n0, n1 in bounds]
            assert max(widths) - min(widths) <= nsplit.ROW_BLOCK
    with pytest.raises(ValueError):
        nsplit.slab_bounds(1024, 2, 2)
    whole = nsplit.seeded_rows(5, 0, 1000, 96, 0.1)
    assert whole.dtype == np.float16 and whole.shape == (1000, 96)
    for world in (2, 3):
        parts = []
        for r in range(world):
            n0, n1 = nsplit.slab_bounds(1000, world, r)
            parts.append(nsplit.seeded_rows(5, n0, n1, 96, 0.1))
        assert np.array_equal(np.concatenate(parts), whole)
    assert not np.array_equal(nsplit.seeded_rows(6, 0, 256, 96, 0.1), whole[:256])
    with pytest.raises(ValueError):
        nsplit.seeded_rows(5, 100, 300, 96, 0.1)
    a0, b0, _ = nsplit.operands(64, 1000, 96, 9, 2, 0)
    a1, b1, _ = nsplit.operands(64, 1000, 96, 9, 2, 1)
    assert np.array_equal(a0, a1) and b0.shape[0] + b1.shape[0] == 1000
    with pytest.raises(ValueError):
        nsplit.assemble([np.zeros((4, 3), np.float16)], [(0, 4)], 4, 4)


NSPLIT_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch
import torch.distributed as dist
from helix_b200 import nsplit
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank = dist.get_rank()
M, N, K = 48, 700, 64
a, b, (n0, n1) = nsplit.operands(M, N, K, 3, 2, rank)
g = object.__new__(nsplit.NSplitGemm)          # host logic only: the slab product is a stand-in computed here
g.M, g.N, g.K, g.world, g.rank, g.n0, g.n1 = M, N, K, 2, rank, n0, n1
g.c = torch.from_numpy((a.astype(np.float32) @ b.astype(np.float32).T).astype(np.float16))
full = g.gather(dist)
a_all, b_all, _ = nsplit.operands(M, N, K, 3, 1, 0)
want = (a_all.astype(np.float32) @ b_all.astype(np.float32).T).astype(np.float16)
print(rank, n0, n1, int(np.array_equal(full, want)))
dist.destroy_process_group()
"""


def test_nsplit_gather_assembles_the_full_product_world_size_2(tmp_path):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "n.py"
    script.write_text(NSPLIT_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stdout=subprocess.PIPE, text=True) for r in (0, 1)]
    outs = [p.communicate(timeout=120)[0].split() for p in procs]
    assert all(p.returncode == 0 for p in procs)
    assert [o[0] for o in outs] == ["0", "1"]
    assert (outs[0][1], outs[0][2], outs[1][1], outs[1][2]) == ("0", "256", "256", "700")
    assert outs[0][3] == "1" and outs[1][3] == "1"


# ----------------------------------------------------------------------------- ablation scripts: selection policies
def test_ablation_selection_policies_on_a_synthetic_dictionary():
    sys.path.insert(0, SCRIPTS)
    try:
        comp = importlib.import_module("Ampere_FP16.benchmark_Ampere_FP16_performance_comparison")
        adap = importlib.import_module("Ampere_FP16.TensorCore_CUDACore_Adaptive")
        curve = importlib.import_module("Ampere_FP16.candidate_performance_curve")
    finally:
        sys.path.remove(SCRIPTS)
    d = synthetic_dict()
    # Static1 never leaves the plain one-CTA kernel; Static2 does not look at the shape
    for shape in [(4096, 4096, 4096), (16, 11008, 4096), (300, 700, 2048)]:
        k1 = comp.cost_model_static1(d, *shape)
        assert k1[0] != 0 and k1[3] == 1 and k1[4] == 0 and k1[5] == 0
    assert comp.cost_model_static2(d, 4096, 4096, 4096) == comp.cost_model_static2(d, 8192, 8192, 2048)
    assert comp.cost_model(d, 4096, 4096, 4096) == costmodel.cost_model(d, 4096, 4096, 4096)
    # GEMV keys are the pick for one right-hand side and never when they are filtered out
    assert adap.cost_model(d, 1, 4096, 1024)[0] == 0
    assert adap.cost_model_without_gemv(d, 1, 4096, 1024)[0] != 0
    assert adap.cost_model_gemv_only(d, 16, 4096, 1024)[0] == 0
    # candidates: ids count kernel keys in dictionary order; GEMV keys only for M <= 8; the best is the model's pick
    cand = curve.candidates(d, 476, 1024, 1024)
    ids = [c[0] for c in cand]
    assert ids == sorted(ids) and all(c[1][0] != 0 for c in cand)
    # (a shape the timing harness overlaps: the scripts' prediction carries that protocol flag)
    assert min(cand, key=lambda c: c[2])[1] == costmodel.cost_model(d, 476, 1024, 1024, overlapped=True)
    assert comp.cost_model(d, 476, 1024, 1024) == costmodel.cost_model(d, 476, 1024, 1024, overlapped=True)
    assert any(c[1][0] == 0 for c in curve.candidates(d, 4, 1024, 1024))


def test_numa_binding_helpers_are_best_effort():
    from helix_b200 import dist_util
    assert dist_util._parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert dist_util._parse_cpulist("") == set()
    before = os.sched_getaffinity(0)
    assert dist_util.bind_to_gpu_numa_node(0, sysfs="/nonexistent") is None     # unreadable topology: nothing changes
    assert os.sched_getaffinity(0) == before


def test_kernel_exe_prints_the_reference_result_line():
    """Token [-8] of the line is the average seconds, as the reference's parsers expect
    (scripts/Ampere_FP16/Ampere_FP16_gemm.py:440; format of src_template/Ampere_FP16/gemm.cu:687-689)."""
    from helix_b200 import kernel_exe
    line = kernel_exe.result_line(4096, 11008, 4096, 1.0e-4, 1.25e-4, 2.0e-4)
    assert line == ("M N K =   4096  11008   4096, Time =   0.00010000   0.00012500   0.00020000 s, "
                    "AVG Performance =  2954.9375 Tflops")
    assert float(line.split()[-8]) == 1.25e-4 and float(line.split()[-2]) == pytest.approx(2954.9375)
    cb = kernel_exe.cublas_line(16, 32, 64, 0.5, 1.25)
    assert float(cb.split()[-4]) == 0.5 and float(cb.split()[-2]) == 1.25      # cublas_f16.cu:101 token positions
    assert kernel_exe.main(["gemm", "1", "2"]) == 2


def test_legacy_port_restates_the_references_pick():
    """oracle/legacy_port.py: executable names <-> dictionary keys, and the reference's cost model
    (scripts/Ampere_FP16/Ampere_FP16_gemm.py:420-430): waves of 108 blocks x probe time, K ignored."""
    from oracle import legacy_port as lp
    assert lp.exe_key("gemm_4_128_256_64_64") == (4, 128, 256, 64, 64, 0)
    assert lp.exe_key("gemm_splitK_3_64_64_32_32") == (3, 64, 64, 32, 32, 1)
    assert lp.exe_key("gemv") == (0, 1, 128, 0, 0, 0) and lp.exe_key("gemv_splitK") == (0, 1, 128, 0, 0, 1)
    assert lp.exe_key("sgemm_128_128_8_8_8_4_4_4") is None and lp.exe_key("im2col") is None
    for name in ("gemm_4_128_256_64_64", "gemm_splitK_3_64_64_32_32", "gemv", "gemv_splitK"):
        assert lp.exe_name(lp.exe_key(name)) == name
    prof = {(3, 128, 128, 64, 64, 0): 1.0e-4, (3, 256, 128, 64, 64, 0): 1.7e-4, (3, 128, 128, 64, 64, 1): 0.6e-4,
            (0, 1, 128, 0, 0, 0): 2.0e-6}
    # 4096^2 outputs: 1024 tiles of 128x128 = 10 waves x 1.0e-4; 512 tiles of 256x128 = 5 waves x 1.7e-4 (the pick);
    # split-K doubles the blocks: 19 waves x 0.6e-4; the GEMV key: 4096 * 32 blocks
    assert lp.reference_cost_model(prof, 4096, 4096, 4096) == (3, 256, 128, 64, 64, 0)
    assert lp.reference_cost_model(prof, 4096, 4096, 64) == (3, 256, 128, 64, 64, 0)      # K plays no part
    assert lp.reference_cost_model(prof, 1, 4096, 4096) == (0, 1, 128, 0, 0, 0)           # one row: 32 blocks, 1 wave
    assert lp.reference_cost_model(prof, 128, 128, 4096) == (0, 1, 128, 0, 0, 0)           # 128 GEMV blocks: 2 waves x 2 us
    del prof[(0, 1, 128, 0, 0, 0)]
    assert lp.reference_cost_model(prof, 128, 128, 4096) == (3, 128, 128, 64, 64, 1)      # one wave each: cheapest probe


def test_cost_model_split_k_modes_and_launch_protocol():
    """Modes 2..4 of a key mean split-K over that many slices (one work item each, all resident at once);
    the prediction describes a lone launch unless the caller says its launches overlap."""
    from helix_b200 import harness
    d = synthetic_dict()
    d[("splitk_overhead", 128)] = (5e-6, 1.2e-6)
    d[("conv_slab_swap", 256)] = 0.5e-6
    d.update({("skinny_fixed",): 2.5e-6, ("wide_gbs_per_sm",): 400.0, ("hbm_wide_gbs",): 5300.0, ("skinny_l2_gbs",): 9300.0})
    k128 = (costmodel.max_stages(128), 128, 128, 1, 0, 0)
    split4 = k128[:5] + (4,)
    assert split4 in costmodel.gemm_keys() and costmodel.is_valid_config(128, 0, 4, 6)
    # 98 tiles x 4 slices do not fit 148 SMs at once: not applicable; 32 tiles x 4 do
    assert costmodel.gemm_time(d, split4, 6272, 256, 2304) == float("inf")
    t1 = costmodel.gemm_time(d, k128, 4096, 128, 8192)
    t4 = costmodel.gemm_time(d, split4, 4096, 128, 8192)
    assert t4 < t1                                    # 32 tiles, 128 slabs each: a quarter of the slabs plus the sum
    assert abs(t4 - (4e-6 + 32 * 0.31e-6 + 5e-6 + 4 * 1.2e-6)) < 1e-9
    # one row block of A: alone, the widest tile on 16 CTAs is bound by its bytes in flight and a split wins;
    # overlapped launches do best unsplit on the widest tile
    lone = costmodel.cost_model(d, 128, 4096, 11008)
    over = costmodel.cost_model(d, 128, 4096, 11008, overlapped=True)
    assert lone[5] != 0 and over[5] == 0                # alone: K is spread over more CTAs (split-K or stream-K)
    wide = (costmodel.max_stages(256), 128, 256, 1, 0, 0)
    assert costmodel.gemm_time(d, wide[:5] + (3,), 128, 4096, 11008) < costmodel.gemm_time(d, wide, 128, 4096, 11008)
    assert costmodel.predicted_time(d, lone, 128, 4096, 11008) < costmodel.predicted_time(d, over, 128, 4096, 11008)
    # swapped convolution tiles only where the caller says the geometry goes through the im2col tensor map
    sw = (costmodel.max_stages(256), 128, 256, 1, 1, 0)
    assert costmodel.gemm_time(d, sw, 25088, 128, 1152, conv=True) == float("inf")
    assert costmodel.gemm_time(d, sw, 25088, 128, 1152, conv="im2col") < float("inf")
    # keys -> configurations
    c = harness.key_to_cfg(split4, prof_dict={("load_group", 128): 3})
    assert (c.split_k, c.stream_k, c.load_group, c.tile_n) == (4, 0, 3, 128)
    c = harness.key_to_cfg(k128[:5] + (1,))
    assert (c.split_k, c.stream_k) == (1, 1)
    assert harness.overlaps(16, 11008, 4096) and not harness.overlaps(4096, 4096, 4096)


def test_stored_channels_of_convolution_inputs():
    """An input of up to four channels is stored with 4 (8-byte pixels) only where the first-layer kernel covers the
    geometry; everything else pads to a multiple of 8.  The sweep's operand shapes follow."""
    from helix_b200 import ops, sweep
    sc = ops.conv_stored_channels
    assert sc(3, 224, 224, 64, 7, 7, 2, 3) == 4          # the ResNet / GoogLeNet first layer
    assert sc(3, 108, 108, 64, 3, 3, 2, 1) == 4
    assert sc(4, 64, 64, 128, 5, 5, 2, 2) == 4
    assert sc(3, 224, 224, 64, 7, 7, 1, 3) == 8          # stride 1
    assert sc(3, 224, 224, 96, 11, 11, 4, 0) == 8        # stride 4 (AlexNet)
    assert sc(3, 224, 224, 32, 7, 7, 2, 3) == 8          # 32 output channels
    assert sc(3, 600, 600, 64, 7, 7, 2, 3) == 8          # output rows longer than 128 pixels
    assert sc(3, 225, 225, 64, 7, 7, 2, 3) == 8          # odd width: rows are not multiples of 16 bytes
    assert sc(3, 224, 224, 64, 7, 8, 2, 3) == 8          # eight taps do not fit beside the alignment shift of an odd pad
    assert sc(1, 161, 700, 32, 5, 20, 2, 0) == 8
    assert sc(5, 224, 224, 64, 7, 7, 2, 3) == 8 and sc(64, 56, 56, 64, 3, 3, 1, 1) == 64 and sc(24, 9, 9, 8, 1, 1, 1, 0) == 24
    a, b, o = sweep.unit_operand_shapes({"kind": "conv", "shape": [32, 3, 224, 224, 64, 7, 7, 2, 3]})
    assert a == (32, 224, 224, 4) and b == (64, 7, 7, 4) and o == (32, 112, 112, 64)


def test_first_layer_kernel_row_ring_never_overwrites_a_row_that_is_still_needed():
    """Restates the row bookkeeping of csrc/conv_f16_stem.cu (RowWalk, the 16-slot ring, the per-slot "last reader"
    and the completion wait the copying warp derives from it) and checks, for many geometries and strips, that every
    item finds its rows in the slots the issuing warps compute, and that a slot is only rewritten after the last item
    that reads its old row is among the items the copying warp has waited for."""
    SLOTS, RING = 16, 16

    def walk(H, Ho, R, pad, t0, t1):
        seg_base = seg_first = count = 0
        prev_hi = -1
        content = [None] * SLOTS          # (image, row) held by each slot
        last_use = [-1] * SLOTS           # item that reads it last
        true_last = {}                    # (image, row) -> last item of the strip that reads it
        for t in range(t0, t1):
            b, oy = divmod(t, Ho)
            for iy in range(max(0, 2 * oy - pad), min(H - 1, 2 * oy - pad + R - 1) + 1):
                true_last[(b, iy)] = t - t0
        for t in range(t0, t1):
            i = t - t0
            b, oy = divmod(t, Ho)
            lo, hi = max(0, 2 * oy - pad), min(H - 1, 2 * oy - pad + R - 1)
            assert lo <= hi
            if i == 0 or oy == 0:
                seg_base, seg_first, new_lo = count, lo, lo
            else:
                new_lo = prev_hi + 1
            if hi >= new_lo:
                count += hi - new_lo + 1
            prev_hi = hi
            index_of = lambda iy: seg_base + iy - seg_first
            need = i - RING // 2
            for iy in range(new_lo, hi + 1):
                need = max(need, last_use[index_of(iy) % SLOTS])
            assert need <= i - 1
            for iy in range(new_lo, hi + 1):
                slot = index_of(iy) % SLOTS
                if content[slot] is not None:
                    assert true_last[content[slot]] <= need, (H, R, pad, t0, t, content[slot])
                content[slot] = (b, iy)
                last_use[slot] = i + min((iy + pad) // 2, Ho - 1) - oy
                assert last_use[slot] >= true_last[(b, iy)]
            slot0 = index_of(lo) % SLOTS
            for k, iy in enumerate(range(lo, hi + 1)):       # what the issuing warp reads: consecutive slots from slot0
                assert content[(slot0 + k) % SLOTS] == (b, iy)

    rng = __import__("random").Random(5)
    for (H, R, pad) in [(224, 7, 3), (20, 7, 3), (64, 3, 1), (64, 5, 2), (40, 8, 2), (33, 4, 0), (9, 2, 0), (11, 8, 7), (7, 7, 3)]:
        Ho = (H + 2 * pad - R) // 2 + 1
        for NB in (1, 3, 40):
            items = NB * Ho
            walk(H, Ho, R, pad, 0, items)
            for _ in range(20):
                a = rng.randrange(items)
                walk(H, Ho, R, pad, a, min(items, a + rng.randrange(1, 60)))
