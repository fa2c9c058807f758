"""GPU: the drop-in scripts end to end (build -> fast profile -> cost model -> sweeps) in a scratch working
directory, the way the reference is driven from its repository root."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = os.path.join(ROOT, "helix_b200", "scripts")


def _run(cwd, script, *args):
    env = dict(os.environ, PYTHONPATH=SCRIPTS)
    out = subprocess.run([sys.executable, os.path.join(SCRIPTS, script), *args], capture_output=True, text=True,
                         env=env, cwd=cwd, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    return out.stdout


@pytest.fixture(scope="module")
def workdir(tmp_path_factory):
    d = tmp_path_factory.mktemp("helix_run")
    _run(d, "build_template.py", "-b", "Ampere_FP16")
    _run(d, "changed_profile.py", "-b", "Ampere_FP16")
    return d


def test_build_and_profile_leave_the_reference_artefacts(workdir):
    assert (workdir / "build" / "bin_fp16" / "MANIFEST").exists()
    text = (workdir / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict").read_text()
    d = eval(text.splitlines()[0])
    assert any(len(k) == 6 and k[0] == 0 for k in d) and any(len(k) == 6 and k[0] != 0 for k in d)
    assert 20.0 < d[("dram_gbs_per_sm",)] < 200.0 and 2000.0 < d[("hbm_gbs",)] < 9000.0


def test_op_level_sweep_prints_the_reference_lines(workdir):
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP16", "-s", "Helix", "--limit", "4")
    lines = [l for l in out.splitlines() if "Helix:" in l]
    assert len(lines) == 4 and lines[0].startswith("2x1024x1024: Helix: ") and lines[0].endswith(" TFLOPS")
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "Conv", "-b", "Ampere_FP16", "-s", "Helix", "--limit", "2")
    assert sum("Helix:" in l for l in out.splitlines()) == 2


def test_vendor_comparators_print_the_reference_lines(workdir):
    """`-s cublas` / `-s cudnn` (context rows beside the B200-native numbers, never on the product path) run and
    print the reference's lines (scripts/Ampere_FP16/benchmark_Ampere_FP16_gemm.py:19-23, ..._conv.py:19-23)."""
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP16", "-s", "cublas", "--limit", "3")
    rows = [l for l in out.splitlines() if ": cublas: " in l]
    assert len(rows) == 3 and all(l.endswith(" TFLOPS") and float(l.split()[-2]) > 0 for l in rows)
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "Conv", "-b", "Ampere_FP16", "-s", "cudnn", "--limit", "3")
    rows = [l for l in out.splitlines() if ": cudnn: " in l]
    assert len(rows) == 3 and all(float(l.split()[-2]) > 0 for l in rows)
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP32", "-s", "cublas", "--limit", "2")
    assert sum(": cublas: " in l for l in out.splitlines()) == 2


def test_sweep_journal_resumes(workdir):
    """--journal: rows are appended per shape and a second run takes them from the file instead of measuring."""
    j = workdir / "sweep.jsonl"
    out1 = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP16", "-s", "Helix", "--limit", "3",
                "--journal", str(j))
    assert len(j.read_text().splitlines()) == 3
    out2 = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP16", "-s", "Helix", "--limit", "4",
                "--journal", str(j))
    assert len(j.read_text().splitlines()) == 4
    first = [l for l in out1.splitlines() if "Helix:" in l]
    again = [l for l in out2.splitlines() if "Helix:" in l]
    assert again[:3] == first and len(again) == 4          # identical numbers: read back, not re-measured


def test_runtime_cost_prints_the_reference_line(workdir):
    out = _run(workdir, "runtime_cost.py", "-b", "Ampere_FP16")
    lines = [l for l in out.splitlines() if l.startswith("The runtime cost of ")]
    assert len(lines) == 7 and "4096x4096x4096" in lines[-1] and "and the op cost is" in lines[-1]


def test_cost_model_prediction_tracks_measurement(workdir):
    """The model's choice must be close to the exhaustive best ("Oracle" vs "Default" in the reference's
    benchmark_Ampere_FP16_performance_comparison.py:44-93) and its time estimate within a factor of two."""
    sys.path.insert(0, ROOT)
    from helix_b200 import costmodel, harness
    d = costmodel.load(str(workdir / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict"))
    for (M, N, K) in [(4096, 4096, 4096), (8192, 768, 3072), (16, 11008, 4096), (2048, 2304, 768)]:
        # the harness overlaps launches for memory-bound shapes: the prediction is asked for that protocol
        key = harness.cost_model(d, M, N, K)
        t_default = harness.time_gemm_f16(M, N, K, harness.key_to_cfg(key, prof_dict=d))
        pred = harness.predicted_time(d, key, M, N, K)
        assert 0.5 <= pred / t_default <= 2.0, (M, N, K, key, pred, t_default)
        best = min(harness.time_gemm_f16(M, N, K, harness.key_to_cfg(k)) for k in costmodel.gemm_keys()
                   if harness.predicted_time(d, k, M, N, K) < float("inf"))
        assert t_default <= 1.3 * best, (M, N, K, key, t_default, best)
    # ... and for one launch alone (the default protocol of the model): one row block of A against long weights
    for (M, N, K) in [(16, 11008, 4096), (128, 4096, 11008)]:
        key = costmodel.cost_model(d, M, N, K)
        t_lone = harness.time_gemm_f16(M, N, K, harness.key_to_cfg(key, prof_dict=d), lone=True)
        pred = costmodel.predicted_time(d, key, M, N, K)
        assert 0.5 <= pred / t_lone <= 2.0, (M, N, K, key, pred, t_lone)
        wide = harness.time_gemm_f16(M, N, K, harness.key_to_cfg((4, 128, 256, 1, 0, 0)), lone=True)
        assert t_lone <= 1.05 * wide, (M, N, K, key, t_lone, wide)     # never worse than the widest unsplit tile


def test_fp32_backend_profile_and_sweep(workdir):
    _run(workdir, "build_template.py", "-b", "Ampere_FP32")
    _run(workdir, "changed_profile.py", "-b", "Ampere_FP32")
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "GEMM", "-b", "Ampere_FP32", "-s", "Helix", "--limit", "2")
    assert sum("Helix:" in l for l in out.splitlines()) == 2
    out = _run(workdir, "benchmark_op_level_eval.py", "-o", "Conv", "-b", "Ampere_FP32", "-s", "Helix", "--limit", "2")
    assert sum("Helix:" in l for l in out.splitlines()) == 2      # column matrix + FFMA GEMM, all three kernels timed


def test_ablation_scripts_run_on_the_profiled_dictionary(workdir):
    """GEMV <-> tensor-core crossover, candidate curve and Oracle/Default/Static comparison
    (reference: TensorCore_CUDACore_Adaptive.py:65-76, candidate_performance_curve.py:6-31,
    benchmark_Ampere_FP16_performance_comparison.py:100-113)."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, SCRIPTS)
    import importlib
    from helix_b200 import costmodel
    adap = importlib.import_module("Ampere_FP16.TensorCore_CUDACore_Adaptive")
    curve = importlib.import_module("Ampere_FP16.candidate_performance_curve")
    comp = importlib.import_module("Ampere_FP16.benchmark_Ampere_FP16_performance_comparison")
    d = costmodel.load(str(workdir / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict"))
    lines = []
    # weights of 128 MiB: streaming time, not launch latency, decides (the script's own list has K = 1024)
    rows = adap.adaptive_table(d, [(1, 16384, 4096), (8, 16384, 4096), (16, 16384, 4096)], out=lines.append)
    assert lines[0].startswith("1x16384x4096: Helix ") and " Gemv " in lines[0] and " GEMM " in lines[0]
    for M, N, K, helix, gemv, gemm in rows:
        assert helix > 0 and gemv > 0 and gemm > 0
        assert helix >= 0.6 * max(gemv, gemm), (M, helix, gemv, gemm)      # the pick is near the better kernel
    assert rows[0][4] > rows[0][5]                # one right-hand side: the GEMV kernel wins
    assert rows[2][5] > rows[2][4]                # sixteen: the tensor-core kernel wins
    lines = []
    best_id, cand = curve.get_all_candidate_performance(d, 128, 512, 1000, out=lines.append)
    assert lines[0].startswith("Best candidate id: ") and len(cand) >= 8 and lines[1].startswith("candidate id: ")
    top = max(c[2] for c in cand)
    assert dict((c[0], c[2]) for c in cand)[best_id] >= 0.5 * top
    lines = []
    (row,) = comp.performance_comparison(d, [(1024, 1024, 1024)], out=lines.append)
    assert "Helix_Oracle:" in lines[0] and "Helix_Static2:" in lines[0]
    _, _, _, oracle, default, s1, s2 = row
    # (three separately timed launches of ~10 us: generous margins against clock noise on a shared box)
    assert oracle >= 0.9 * max(default, s1, s2) and default >= 0.65 * oracle, row


def test_op_level_list_sampled_parity_with_the_models_pick(workdir):
    """Every 29th shape of the op-level GEMM list (plus the shapes whose K is no multiple of 8) computed with
    the configuration the cost model picks -- GEMV keys included -- and checked against the oracle on sampled
    rows: the sweep reports numbers for results that are right."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, SCRIPTS)
    import numpy as np
    import torch
    from helix_b200 import costmodel, harness, ops
    from oracle import api as oracle
    from tests import util
    from utils.get_benchmark_shape_list import get_gemm_op_MNKList
    oracle.build()
    d = costmodel.load(str(workdir / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict"))
    shapes = get_gemm_op_MNKList()
    picked = shapes[::29] + [s for s in shapes if s[2] % 8][::7]
    # the extremes of the DeepBench- and GNN-derived tables: K = 500 000 against one or four columns, 1.9 M rows
    # against 16 columns with K = 66, K = 29, three to seven columns
    extremes = [(512, 1, 500000), (1024, 4, 500000), (1889542, 16, 66), (43466, 16, 29), (2708, 16, 1433),
                (7680, 2, 2560), (35, 700, 2048)] + [s for s in shapes if s[1] in (3, 6, 7)][:3]
    assert all(e in shapes for e in extremes)
    picked += extremes
    kinds = set()
    for idx, (M, N, K) in enumerate(picked):
        rng = np.random.default_rng(1000 + idx)
        s = np.float32(1.0 / np.sqrt(K))
        a = (rng.standard_normal((M, K), dtype=np.float32) * s).astype(np.float16)
        b = (rng.standard_normal((N, K), dtype=np.float32) * s).astype(np.float16)
        Kp = (K + 7) // 8 * 8                      # leading dimensions follow the 16-byte rule; zero columns add nothing
        ad = torch.zeros((M, Kp), dtype=torch.float16, device="cuda")
        bd = torch.zeros((N, Kp), dtype=torch.float16, device="cuda")
        ad[:, :K] = torch.from_numpy(a).cuda()
        bd[:, :K] = torch.from_numpy(b).cuda()
        key = costmodel.cost_model(d, M, N, K)
        cfg = harness.key_to_cfg(key)
        if key[0] == 0:
            kinds.add("gemv")
            if M <= N:
                out = torch.empty((M, N), dtype=torch.float16, device="cuda")
                ops.run(ops.launch_gemv_f16(bd, ad, out, cfg))
            else:
                out = torch.empty((M, N), dtype=torch.float16, device="cuda")
                ops.run(ops.launch_gemv_f16(ad, bd, out, cfg, out_transposed=True))
        else:
            kinds.add("pair" if key[3] == 2 else ("swap" if key[4] else ("streamk" if key[5] else "plain")))
            out = ops.gemm_f16(ad, bd, cfg=cfg)
        torch.cuda.synchronize()
        ops.check_status()
        rows = sorted({0, M // 3, M // 2, M - 1})
        _, ref32 = oracle.hgemm_naive(np.ascontiguousarray(a[rows]), b)
        util.assert_f16_close(out[rows].cpu().numpy(), ref32, f"{M}x{N}x{K} with {key}")
    assert {"gemv", "pair"} <= kinds and len(kinds) >= 3, kinds


def test_conv_op_level_list_sampled_parity_with_the_models_pick(workdir):
    """Every 53rd layer of the op-level convolution list (3, 24, 32 ... 832 input channels, 1x1 to 11x11
    filters, strides 1, 2, 4) run the way harness.time_conv_f16 runs it -- channels padded to a multiple of
    8, the cost model's key -- with its first and last image checked against the oracle."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, SCRIPTS)
    import numpy as np
    import torch
    from helix_b200 import costmodel, harness, ops
    from oracle import api as oracle
    from tests import util
    from utils.get_benchmark_shape_list import get_conv_op_shape_list
    oracle.build()
    d = costmodel.load(str(workdir / "build" / "prof_dict" / "Ampere_FP16_cost_model.dict"))
    layers = get_conv_op_shape_list()
    # plus the DeepBench speech layers: one input channel, 5 x 20 and 5 x 10 filters, stride 2
    speech = [(1, 1, 161, 700, 32, 5, 20, 2, 0), (4, 32, 79, 341, 32, 5, 10, 2, 0)]
    assert all(l in layers for l in speech)
    for idx, (B, IC, H, W, OC, kH, kW, stride, pad) in enumerate(layers[::53] + speech):
        rng = np.random.default_rng(2000 + idx)
        C = ops.conv_stored_channels(IC, H, W, OC, kH, kW, stride, pad)
        x = np.zeros((B, H, W, C), np.float16)
        w = np.zeros((OC, kH, kW, C), np.float16)
        x[..., :IC] = rng.uniform(-1, 1, (B, H, W, IC)).astype(np.float16)
        w[..., :IC] = (rng.standard_normal((OC, kH, kW, IC), dtype=np.float32) * np.float32((2.0 / (IC * kH * kW)) ** 0.5)).astype(np.float16)
        Ho, Wo = ops.conv_out_hw(H, W, kH, kW, stride, pad)
        M, N, K = B * Ho * Wo, OC, IC * kH * kW
        as_gemm = kH == 1 and kW == 1 and stride == 1 and pad == 0
        key = costmodel.cost_model(d, M, N, (K + 7) // 8 * 8, 1, conv=not as_gemm)
        if key is None or key[0] == 0:
            key = (costmodel.max_stages(128), 128, 128, 1, 0, 0)       # as harness.conv_f16_result falls back
        y = ops.conv2d_f16_nhwc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), stride, pad,
                                cfg=harness.key_to_cfg(key, conv=True))
        torch.cuda.synchronize()
        ops.check_status()
        for img in sorted({0, B - 1}):
            _, y32 = oracle.conv2d_nhwc_f16(x[img:img + 1], w, stride, pad)
            util.assert_f16_close(y[img:img + 1].cpu().numpy(), y32, f"conv {(B, IC, H, W, OC, kH, kW, stride, pad)} image {img} with {key}")


def test_conv_op_level_first_layers_parity():
    """Every layer of the op-level convolution list that is stored with 4 channels (the 7 x 7 / 2 first layer at
    batch 1 ... 64 and a 3 x 3 / 2 one) through the first-layer kernel: first and last image against the oracle."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, SCRIPTS)
    import numpy as np
    import torch
    from helix_b200 import ops
    from oracle import api as oracle
    from tests import util
    from utils.get_benchmark_shape_list import get_conv_op_shape_list
    oracle.build()
    layers = sorted({l for l in get_conv_op_shape_list() if ops.conv_stored_channels(*l[1:]) == 4})
    assert len(layers) >= 19
    for idx, (B, IC, H, W, OC, kH, kW, stride, pad) in enumerate(layers):
        rng = np.random.default_rng(3000 + idx)
        x = np.zeros((B, H, W, 4), np.float16)
        w = np.zeros((OC, kH, kW, 4), np.float16)
        x[..., :IC] = rng.uniform(-1, 1, (B, H, W, IC)).astype(np.float16)
        w[..., :IC] = (rng.standard_normal((OC, kH, kW, IC), dtype=np.float32) * np.float32((2.0 / (IC * kH * kW)) ** 0.5)).astype(np.float16)
        y = ops.conv2d_f16_nhwc(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), stride, pad)
        torch.cuda.synchronize()
        ops.check_status()
        for img in sorted({0, B - 1}):
            _, y32 = oracle.conv2d_nhwc_f16(x[img:img + 1], w, stride, pad)
            util.assert_f16_close(y[img:img + 1].cpu().numpy(), y32, f"first layer {(B, IC, H, W, OC, kH, kW, stride, pad)} image {img}")
