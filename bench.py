#!/usr/bin/env python
"""Benchmark of the Helix hot path on B200: the model-level fp16 GEMM / convolution sweep.

Work list: INSTANCES copies (distinct seeded data) of the model-level sweep -- every GEMM of a BERT-base
encoder at batch 16 / seq 512 and the 53 ResNet-50 convolutions at batch 32, 125 independent units and
1.81 TFLOP per copy.  With N GPUs the list is partitioned over the ranks (longest-processing-time-first on
a roofline estimate, no collective in the data path); the job's time is the slowest rank's, so the figure
is strong scaling of a fixed list.  One step = PASSES passes over the list, so that the default timed region
lasts seconds, not milliseconds.  Prints ONE JSON line (rank 0).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl helix|reference]

`--impl reference` times the CPU restatement of the reference's x86 template (its own CPU path is TVM
generated and cannot be built here) with all host threads, one pass over one copy of the sweep per step.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fp16_gemm_conv_sweep_tflops"
UNIT = "TFLOP/s"
INSTANCES = 8        # copies of the model-level sweep in the work list
PASSES = 6           # passes over the list per step


def workload_text():
    return ("model-level sweep: BERT-base b16 s512 (72 GEMMs incl. batched QK^T/PV) + ResNet-50 b32 224x224 "
            "(53 convs), work list = %d seeded copies (%d units)" % (INSTANCES, INSTANCES * 125))


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


def host_threads():
    """Threads the CPU arm uses: the CPUs this process may run on.  Passed to the oracle explicitly, so that an
    OMP_NUM_THREADS=1 inherited from a launcher cannot shrink it."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the x86 template on one copy of the sweep
# ----------------------------------------------------------------------------------------------
class CpuSweep:
    """One copy of the model-level sweep as the reference's x86 backend would run it: every unit an fp32
    GEMM (a convolution as M = B*Ho*Wo, N = OC, K = IC*kH*kW, the reference's own mapping), the parallel
    packed schedule with the tiling its profile-driven chooser picks per shape.  Repeated shapes share
    their operand buffers."""

    def __init__(self, threads):
        import numpy as np
        from helix_b200 import workloads
        from oracle import api, x86_tiling
        self.api, self.threads = api, threads
        self.prof, self.prof_info = x86_tiling.profile()
        self.calls = []       # (a, b, c, tiling, count)
        self.flops = 0.0
        shapes = {}
        for u in workloads.model_level_sweep():
            s = u["shape"]
            if u["kind"] == "gemm":
                M, N, K = s[:3]
                cnt = s[3] if len(s) > 3 else 1
            else:
                B, IC, H, W, OC, kh, kw, stride, pad = s
                Ho, Wo = (H + 2 * pad - kh) // stride + 1, (W + 2 * pad - kw) // stride + 1
                M, N, K, cnt = B * Ho * Wo, OC, IC * kh * kw, 1
            shapes[(M, N, K)] = shapes.get((M, N, K), 0) + cnt
            self.flops += 2.0 * M * N * K * cnt
        rng = np.random.default_rng(4)
        self.tilings = {}
        for (M, N, K), cnt in shapes.items():
            s = np.float32(1.0 / np.sqrt(K))
            a = rng.standard_normal((M, K), dtype=np.float32) * s
            b = rng.standard_normal((K, N), dtype=np.float32) * s
            tl = x86_tiling.get_tiling(self.prof, M, N, K, threads)
            self.tilings[(M, N, K)] = tl
            self.calls.append((a, b, np.empty((M, N), np.float32), tl, cnt))

    def one_pass(self):
        t0 = time.perf_counter()
        for a, b, c, tl, cnt in self.calls:
            for _ in range(cnt):
                self.api.sgemm_parallel(a, b, tiling=tl, threads=self.threads, fma=True, out=c)
        return time.perf_counter() - t0

    def sample_text(self, seconds):
        return ("one pass over one copy of the sweep: all 125 units (%d distinct GEMM shapes, convolutions as "
                "M=B*Ho*Wo N=OC K=IC*kH*kW at batch 32), fp32 x86-template restatement with fused multiply-add, "
                "tiling per shape from the restated profile (%d register blocks kept, best single-thread probe "
                "%.0f GFLOP/s against the reference's 0.6 x 153), %.2f TFLOP in %.1f s"
                % (len(self.calls), self.prof_info["register_blocks_kept"], self.prof_info["best_probe_gflops"],
                   self.flops / 1e12, seconds))


def bench_reference(args, rank, world):
    if rank != 0:
        return
    cores = host_threads()
    if cores < 2 and (os.cpu_count() or 1) >= 2:
        raise SystemExit("reference arm: only %d usable CPU of %d" % (cores, os.cpu_count()))
    cpu = CpuSweep(cores)
    times = []
    for i in range(args.warmup + args.steps):
        dt = cpu.one_pass()
        if i >= args.warmup:
            times.append(dt)
    avg = sum(times) / len(times)
    value = cpu.flops / avg / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": avg * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_text(), "step": "one pass over one copy of the sweep (1/%d of the list, every "
                                                  "distinct unit in its real count)" % INSTANCES},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "gflops_per_core": value * 1e3 / cores, "sample": cpu.sample_text(avg)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="helix_clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, mx, power = [], set(), None, []
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1]))
                        mx = float(p[2])
                        power.append(float(p[3]))
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         p[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        if sm:
            # the samples taken under load: the sampler also sees the idle edges of the region
            busy = sorted(s for s, w in zip(sm, power) if w >= 0.5 * max(power)) or sorted(sm)
            out["sm_mhz"] = busy[len(busy) // 2]
            out["sm_max_mhz"] = mx
            out["sm_min_mhz_seen"] = min(sm)
            out["power_w_max"] = max(power)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def unit_estimate(u):
    """Roofline estimate (seconds) of one unit, the cost the work list is partitioned by."""
    from helix_b200 import workloads
    return max(workloads.unit_flops(u) / 1.0e15, workloads.unit_bytes(u) / 5.0e12) + 4e-6


def work_list():
    from helix_b200 import workloads
    units = []
    for inst in range(INSTANCES):
        for u in workloads.model_level_sweep():
            v = dict(u)
            v["name"] = "copy%d.%s" % (inst, u["name"])
            v["index"] = len(units)
            units.append(v)
    return units


def per_config_table(peaks):
    """The configurations the baseline names, one compact row each: [microseconds, rate, fraction of peak]
    (GB/s against the measured HBM copy rate for memory-bound rows, TFLOP/s against the measured burst tensor
    peak or the nominal FFMA peak otherwise).  Two protocols where they differ: "alone" = ordered launches on
    one buffer set, each waiting for its predecessor (what a caller's single call sees, and how the vendor
    comparators are timed); "overlapped" = launches on distinct buffer sets flagged independent, which share
    the machine (throughput of a sweep of such calls)."""
    import torch
    from helix_b200 import datagen, ops
    from helix_b200._lib import LAUNCH_INDEPENDENT, LAUNCH_STATIC_A, OP_GEMM_F16
    dev = "cuda"
    out = {}
    r3 = lambda us, rate, frac: [round(us, 2), round(rate, 1), round(frac, 3)]
    # Every row is a kernel timed alone against a burst peak, so every row starts from a rested GPU: after a
    # stretch at the power cap the clocks stay low for a while (a table measured back to back showed 1100 MHz
    # samples and rows 20-50 % slower than the same kernels measured one at a time).
    def timed(ls, warmup=3, iters=20):
        torch.cuda.synchronize()
        time.sleep(0.5)
        return ops.time_launches(ls, warmup=warmup, iters=iters, use_graph=True)
    # C2: fp16 GEMV 4096 x 4096, m = 1: twelve rotating W buffers (12 x 32 MiB > 2 x L2) in three
    # launch-ordering modes, plus one 268 MB matrix (16384 x 8192) streamed by chains of ordered launches
    rows = K = 4096
    ws = [torch.randn(rows, K, device=dev, dtype=torch.float16) * 0.02 for _ in range(12)]
    x = torch.randn(1, K, device=dev, dtype=torch.float16)
    ys = [torch.empty(1, rows, device=dev, dtype=torch.float16) for _ in ws]
    ls = [ops.launch_gemv_f16(w, x, y) for w, y in zip(ws, ys)]
    gemv_bytes = rows * K * 2 + K * 2 + rows * 2
    g = {}
    for name, flag in (("independent", LAUNCH_INDEPENDENT), ("static_weights", LAUNCH_STATIC_A), ("ordered", 0)):
        for l in ls:
            l.flags = flag
        avg, _, _ = timed(ls, warmup=5, iters=50)
        gb = gemv_bytes / avg / 1e9
        g[name] = r3(avg * 1e6, gb, gb / peaks["hbm_gbs"])
    del ws, ys, ls
    big = [torch.randn(16384, 8192, device=dev, dtype=torch.float16) * 0.02 for _ in range(2)]
    xb = torch.randn(1, 8192, device=dev, dtype=torch.float16)
    yb = [torch.empty(1, 16384, device=dev, dtype=torch.float16) for _ in big]
    ls = [ops.launch_gemv_f16(w, xb, y) for w, y in zip(big, yb)]
    avg, _, _ = timed(ls, warmup=3, iters=20)
    gb = (16384 * 8192 * 2 + 8192 * 2 + 16384 * 2) / avg / 1e9
    g["16384x8192_ordered"] = r3(avg * 1e6, gb, gb / peaks["hbm_gbs"])
    del big, yb, ls
    out["gemv_4096x4096_m1 [us, GB/s, of_hbm]"] = g
    # C3: dense fp16 GEMMs.  Memory-bound shapes (one row block of A): the library's choice alone on one buffer
    # set, and the widest tile without split-K overlapped on eight buffer sets (8 x 90 MB > 2 x L2)
    c3 = {}
    for (M, N, K) in datagen.C3_SHAPES:
        by = 2.0 * (M * K + N * K + M * N)
        fl = 2.0 * M * N * K
        membound = fl / by <= 300
        nbuf = 8 if membound else 1
        bufs = [(torch.randn(M, K, device=dev, dtype=torch.float16) / K ** 0.5,
                 torch.randn(N, K, device=dev, dtype=torch.float16) / K ** 0.5,
                 torch.empty(M, N, device=dev, dtype=torch.float16)) for _ in range(nbuf)]
        a, b, c = bufs[0]
        avg, _, _ = timed([ops.launch_gemm_f16(a, b, c)] * 4, warmup=3, iters=20)
        if membound:
            gbs = by / avg / 1e9
            row = {"alone": r3(avg * 1e6, gbs, gbs / peaks["hbm_gbs"])}
            wide = ops.make_cfg(OP_GEMM_F16, 128, 256, 64)
            ls = [ops.launch_gemm_f16(a, b, c, wide) for a, b, c in bufs]
            for l in ls:
                l.flags = LAUNCH_INDEPENDENT
            avg, _, _ = timed(ls, warmup=3, iters=20)
            gbs = by / avg / 1e9
            row["overlapped"] = r3(avg * 1e6, gbs, gbs / peaks["hbm_gbs"])
            row["unit"] = "GB/s"
            c3["%dx%dx%d" % (M, N, K)] = row
        else:
            tf = fl / avg / 1e12
            c3["%dx%dx%d" % (M, N, K)] = r3(avg * 1e6, tf, tf / peaks["tflops"]) + ["TFLOP/s"]
        del bufs, a, b, c
    out["gemm_f16 [us, rate, of_peak]"] = c3
    # C4: ResNet-style convolutions at batch 32, each rated against its own floor max(flops/peak, bytes/hbm);
    # fourth figure: microseconds per launch when four launches on distinct buffers overlap
    c4 = {}
    # plus the first layer of the model-level CNN (3 channels stored as 4: the raw-row kernel), flops counted on 3
    for layer in list(datagen.C4_LAYERS) + [(32, 3, 224, 224, 64, 7, 7, 2, 3)]:
        B, IC, H, W, OC, kh, kw, s, p = layer
        C = ops.conv_stored_channels(IC, H, W, OC, kh, kw, s, p)
        Ho, Wo = ops.conv_out_hw(H, W, kh, kw, s, p)
        ls = []
        for _ in range(4):
            xx = torch.rand(B, H, W, C, device=dev, dtype=torch.float16) * 2 - 1
            ww = torch.randn(OC, kh, kw, C, device=dev, dtype=torch.float16) * (2.0 / (C * kh * kw)) ** 0.5
            yy = torch.empty(B, Ho, Wo, OC, device=dev, dtype=torch.float16)
            ls.append(ops.launch_conv2d_f16(xx, ww, yy, s, p))
        avg, _, _ = timed([ls[0]] * 4, warmup=3, iters=20)
        for l in ls:
            l.flags = LAUNCH_INDEPENDENT
        over, _, _ = timed(ls, warmup=3, iters=20)
        fl = 2.0 * B * Ho * Wo * OC * IC * kh * kw
        by = 2.0 * (xx.numel() + ww.numel() + yy.numel())
        floor = max(fl / (peaks["tflops"] * 1e12), by / (peaks["hbm_gbs"] * 1e9))
        c4["x".join(map(str, layer))] = r3(avg * 1e6, fl / avg / 1e12, floor / avg) + [round(over * 1e6, 2)]
        del ls
    out["conv_f16 [us, TFLOP/s, of_roofline, us_overlapped]"] = c4
    # C1: fp32 FFMA GEMM 1024^3 (the configuration the reference's CPU template runs), nominal FFMA peak 74.4
    c1 = {}
    for n in (1024, 2048, 4096):
        a = torch.rand(n, n, device=dev) * 2 - 1
        b = torch.rand(n, n, device=dev) * 2 - 1
        c = torch.empty(n, n, device=dev)
        avg, _, _ = timed([ops.launch_gemm_f32(a, b, c)] * 4, warmup=3, iters=10)
        tf = 2.0 * n ** 3 / avg / 1e12
        c1[str(n)] = r3(avg * 1e6, tf, tf / 74.4)
        del a, b, c
    out["gemm_f32 [us, TFLOP/s, of_ffma_nominal_74.4]"] = c1
    # fp32 GEMV 8192 x 8192 (268 MB of weights per launch, two buffers)
    wf = [torch.rand(8192, 8192, device=dev) * 2 - 1 for _ in range(2)]
    xf = torch.rand(1, 8192, device=dev) * 2 - 1
    yf = [torch.empty(1, 8192, device=dev) for _ in wf]
    avg, _, _ = timed([ops.launch_gemv_f32(w, xf, y) for w, y in zip(wf, yf)], warmup=3, iters=20)
    gb = (8192 * 8192 * 4 + 2 * 8192 * 4) / avg / 1e9
    out["gemv_f32_8192x8192_m1 [us, GB/s, of_hbm]"] = r3(avg * 1e6, gb, gb / peaks["hbm_gbs"])
    del wf, yf
    return out


def extras(peaks):
    """Further context rows: true-fp32 convolutions and the vendor libraries on the same box."""
    import torch
    from helix_b200 import datagen, harness, ops
    out = {}
    c32 = {}
    for layer in datagen.C4_LAYERS[:2] + datagen.C4_LAYERS[3:4]:
        B, C, H, W, OC, kh, kw, s, p = layer
        torch.cuda.synchronize()
        time.sleep(0.5)           # every row starts from a rested GPU (see per_config_table)
        t = harness.time_conv_f32(*layer)
        Ho, Wo = ops.conv_out_hw(H, W, kh, kw, s, p)
        tf = 2.0 * B * Ho * Wo * OC * C * kh * kw / t / 1e12
        c32["x".join(map(str, layer))] = {"us": round(t * 1e6, 1), "TFLOP/s": round(tf, 1), "of_ffma_nominal_74.4": round(tf / 74.4, 3)}
    out["conv_f32"] = c32
    # vendor comparators (context only, never on the product path): cuBLAS fp16 with fp32 accumulate, cuDNN NHWC
    comp = {}
    try:
        for (M, N, K) in datagen.C3_SHAPES:
            torch.cuda.synchronize()
            time.sleep(0.5)
            ms, tf = harness.cublas_gemm_result(M, N, K)
            comp["cublas %dx%dx%d" % (M, N, K)] = {"us": round(ms * 1e3, 1), "TFLOP/s": round(tf, 1)}
        for layer in datagen.C4_LAYERS:
            torch.cuda.synchronize()
            time.sleep(0.5)
            ms, tf = harness.cudnn_conv_result(*layer)
            comp["cudnn " + "x".join(map(str, layer))] = {"us": round(ms * 1e3, 1), "TFLOP/s": round(tf, 1)}
    except Exception as exc:     # a comparator that fails does not fail the benchmark
        comp["error"] = repr(exc)
    out["comparators"] = comp
    return out


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, averaged over the launches of one
# pass over one copy of the sweep) for each kernel, from single-pass ncu captures; the capture commands are
# in profiles/bench_sweep_launch_list.md.  Kernels that capture did not list report null.
SWEEP_DRAM_BYTES_PER_LAUNCH = {
    "gemm_f16_tc2_kernel<256>": 15810162, "gemm_f16_tc2_kernel<192>": 34526677,
    "gemm_f16_tc_kernel<256,0>": 30764491, "gemm_f16_tc_kernel<64,0>": 68126530,
    "gemm_f16_tc_kernel<128,0>": 14688633, "gemm_f16_tc_kernel<64,1>": 26433792,
    "conv_f16_stem_kernel<4>": 13823700,   # profiles/conv_f16_stem_kernel_7x7_c3_224x224.md
    "conv_f16_rows_kernel": 12970000,      # profiles/conv_f16_rows_kernel_3x3_c64_56x56.md
}


def kernel_breakdown(sw, ops, limit_units=125):
    """Time the launches of one copy of the sweep grouped by the kernel they resolve to in the sweep (CUDA-graph
    replay, events on the launching stream, each group alone on the whole machine with the sweep's own tile
    choice): launches, seconds and algorithmic flop / bytes per group."""
    from helix_b200 import workloads
    import ctypes
    import torch
    from helix_b200._lib import Launch
    groups = {}
    for u, l0 in list(zip(sw.units, sw.launches))[:limit_units]:
        l = Launch()
        ctypes.memmove(ctypes.byref(l), ctypes.byref(l0), ctypes.sizeof(Launch))
        # the kernel and tile the sweep really launches for this unit (chosen for its share of the SMs), made
        # explicit, then given the whole machine: the groups carry the names a profiler sees in the sweep
        if not (l.cfg.tile_m or l.cfg.tile_n):
            chosen = ops.default_config(l)
            chosen.max_ctas = l.cfg.max_ctas
            l.cfg = chosen
        ops.limit_ctas(l, 0)
        g = groups.setdefault(ops.kernel_name(l), {"launches": [], "flop": 0.0, "bytes": 0.0})
        g["launches"].append(l)
        g["flop"] += workloads.unit_flops(u)
        g["bytes"] += workloads.unit_bytes(u)
    out = {}
    for name, g in groups.items():
        torch.cuda.synchronize()
        time.sleep(0.5)           # each group starts from a rested GPU: it is rated against the burst peak
        avg, _, _ = ops.time_launches(g["launches"], warmup=3, iters=10, use_graph=True)
        n = len(g["launches"])
        out[name] = {"launches": n, "us": avg * n * 1e6, "flop": g["flop"], "bytes": g["bytes"]}
    total = sum(v["us"] for v in out.values())
    for v in out.values():
        v["share"] = v["us"] / total
        v["TFLOP/s"] = v["flop"] / (v["us"] * 1e-6) / 1e12
    return out


def self_check(sw):
    """Untimed: a few units of what was just timed (outputs of the last replay) against the CPU oracle.
    Raises when one is outside the fp16 tolerance (relative Frobenius error 2e-3)."""
    import numpy as np
    from oracle import api as oracle
    want = ["bert.l0.qkv", "bert.l0.qk", "bert.l0.pv", "resnet50.stem", "resnet50.s1b0.conv2", "resnet50.s4b2.conv3"]
    checked, worst = 0, 0.0
    for u, (a, b, out) in zip(sw.units, sw.tensors):
        tag = u["name"].split(".", 1)[1]
        if tag not in want:
            continue
        want.remove(tag)
        s = u["shape"]
        if u["kind"] == "gemm" and len(s) == 3:
            got, (_, ref) = out.cpu().numpy(), oracle.hgemm_fast(a.cpu().numpy(), b.cpu().numpy())
        elif u["kind"] == "gemm":
            got, (_, ref) = out[0].cpu().numpy(), oracle.hgemm_naive(a[0].cpu().numpy(), b[0].cpu().numpy())
        else:
            got = out[:1].cpu().numpy()
            _, ref = oracle.conv2d_nhwc_f16(np.ascontiguousarray(a[:1].cpu().numpy()), b.cpu().numpy(), s[7], s[8])
        err = float(np.linalg.norm(got.astype(np.float64) - ref) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30))
        if not np.isfinite(err) or err > 2e-3:
            raise SystemExit("bench self-check failed: %s relative Frobenius error %.3e" % (u["name"], err))
        worst = max(worst, err)
        checked += 1
    return checked, worst


def bench_helix(args, rank, world, local_rank):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from helix_b200 import dist_util, ops, sweep, workloads
    peaks = read_peaks()
    numa_cpus = dist_util.bind_to_gpu_numa_node(local_rank) if world > 1 else None

    # The per-configuration rows are single kernels rated against burst peaks: they are measured first, on a GPU
    # that has not yet run into its power cap (after the seconds-long sweep below the clocks stay low for a while:
    # a table measured then showed 1100 MHz samples and 10-50 % longer times than the same kernels on a fresh GPU).
    table = table_extras = None
    if world == 1 and not args.no_extras:
        xs = ClockSampler(local_rank)
        xs.start()
        table = per_config_table(peaks)
        table_extras = extras(peaks)
        table_extras["clocks"] = xs.stop()
        torch.cuda.empty_cache()

    # this rank's share of the fixed work list
    units = work_list()
    total_flops = sum(workloads.unit_flops(u) for u in units)
    parts = workloads.lpt_partition([unit_estimate(u) for u in units], world)
    mine = [units[i] for i in parts[rank]]
    sw = sweep.Sweep(mine, seed=4000, lanes=args.lanes, seeds=[u["index"] for u in mine])
    launches_per_pass = sw.step()          # outside any capture: sets function attributes, fills the tensor-map cache
    torch.cuda.synchronize()
    ops.check_status()

    graph = None
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            sw.step()
        graph = g
    except Exception:
        graph = None
        torch.cuda.synchronize()

    # the per-kernel groups are timed alone, before the seconds-long region drives the GPU into its power cap
    groups = kernel_breakdown(sw, ops) if rank == 0 else None
    ops.check_status()

    def one_step():
        for _ in range(args.passes):
            if graph is not None:
                graph.replay()
            else:
                sw.step()

    for _ in range(args.warmup):
        one_step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    dist_util.barrier(dist)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    dist_util.barrier(dist)
    own_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status()
    ms = dist_util.max_over_ranks(own_ms, dist, "cuda")
    rank_ms = dist_util.gather_floats(own_ms, dist, "cuda")
    ms_per_step = ms / args.steps
    value = total_flops * args.passes / (ms_per_step * 1e-3) / 1e12

    # end to end: this rank's units with pinned host operands in and results out, every pass
    hs = sweep.HostSweep(sw)
    e2e_passes = max(1, min(args.steps, 3))
    hs.step()
    hs.finish()
    dist_util.barrier(dist)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_passes):
        hs.step()
    hs.finish()
    e2e_own = (time.perf_counter() - t0) / e2e_passes
    e2e_s = dist_util.max_over_ranks(e2e_own, dist, "cuda")
    e2e_value = total_flops / e2e_s / 1e12
    h2d_total = dist_util.sum_over_ranks(hs.h2d_bytes, dist, "cuda")
    d2h_total = dist_util.sum_over_ranks(hs.d2h_bytes, dist, "cuda")
    ops.check_status()
    del hs

    # secondary figure: every rank runs one whole copy of the sweep (independent replicas)
    replica = None
    if world > 1:
        one_copy = sweep.Sweep(workloads.model_level_sweep(), seed=4000 + rank, lanes=args.lanes)
        one_copy.step()
        torch.cuda.synchronize()
        dist_util.barrier(dist)
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(10):
            one_copy.step()
        r1.record()
        torch.cuda.synchronize()
        rep_ms = dist_util.max_over_ranks(r0.elapsed_time(r1) / 10, dist, "cuda")
        replica = {"value": one_copy.flops * world / (rep_ms * 1e-3) / 1e12, "ms_per_pass": rep_ms,
                   "what": "every rank one whole copy of the sweep on its own data (weak scaling, eager launches)"}
        del one_copy
        ops.check_status()

    # one oversized GEMM split along N (no collective in the timed region), N > 1 only
    nsplit_row = None
    if world > 1:
        from helix_b200 import nsplit
        import numpy as np
        M, K = 8192, 8192
        N = 16384 * world
        gsp = nsplit.NSplitGemm(M, N, K, 2, world, rank)
        for _ in range(3):
            gsp.step()
        torch.cuda.synchronize()
        dist_util.barrier(dist)
        n0e, n1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n0e.record()
        for _ in range(10):
            gsp.step()
        n1e.record()
        torch.cuda.synchronize()
        ns_ms = dist_util.max_over_ranks(n0e.elapsed_time(n1e) / 10, dist, "cuda")
        digest = float(gsp.c.float().abs().sum().item())
        nsplit_row = {"M": M, "N": N, "K": K, "ms": ns_ms, "TFLOP/s": 2.0 * M * N * K / (ns_ms * 1e-3) / 1e12,
                      "checksum_abs_sum_all_slabs": dist_util.sum_over_ranks(digest, dist, "cuda"),
                      "collectives_in_timed_region": 0}
        del gsp
        ops.check_status()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    per_gpu = value / world
    top = max(groups, key=lambda k: groups[k]["share"])
    tg = groups[top]
    checked, worst_err = self_check(sw)
    pass_ms = ms_per_step / args.passes
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 in / f32 accumulate", "data": "synthetic",
        "config": {"workload": workload_text(), "step": "%d passes over the work list (%.2f TFLOP per pass)" % (args.passes, total_flops / 1e12),
                   "units_this_rank": len(mine), "cache": "operands of one pass on rank 0 total %.1f GB (> L2), one buffer set per unit" % (sw.bytes / 1e9),
                   "cuda_graph": graph is not None,
                   "parallelism": "fixed work list partitioned over %d GPU(s) by LPT on a roofline estimate; no collective" % world,
                   "lanes": "%d concurrent launch chains per GPU, each launch limited to 1/%d of the SMs" % (args.lanes, args.lanes),
                   "host_numa_binding": ("rank 0 bound to %d CPUs next to its GPU" % len(numa_cpus)) if numa_cpus else "none"},
        "ms_per_pass": pass_ms,
        "rank_idle_frac": [round(1.0 - t / ms, 4) for t in rank_ms],
        "checked_units": checked, "check_worst_rel_fro": worst_err,
        "roofline": {"bound": "tensor", "achieved": tg["TFLOP/s"], "peak": peaks["tflops"], "unit": "TFLOP/s",
                     "frac": tg["TFLOP/s"] / peaks["tflops"],
                     "traffic": SWEEP_DRAM_BYTES_PER_LAUNCH.get(top),
                     "traffic_source": "constant from a single-pass ncu capture of one sweep pass (profiles/bench_sweep_launch_list.md), not measured by this run",
                     "kernel": top, "launches_per_copy": tg["launches"], "share_of_copy": tg["share"],
                     "us_per_launch": tg["us"] / tg["launches"],
                     "algorithmic_flop_per_launch": tg["flop"] / tg["launches"],
                     "algorithmic_bytes_per_launch": tg["bytes"] / tg["launches"],
                     "peak_source": peaks["source"] + " burst bf16 cuBLAS (the group is timed alone for ~10 ms before the sustained region); sustained %.0f" % peaks["tflops_sustained"],
                     "whole_sweep": {"achieved_per_gpu": per_gpu, "frac_of_sustained": per_gpu / peaks["tflops_sustained"],
                                     "frac_of_burst": per_gpu / peaks["tflops"], "timed_region_s": ms * 1e-3,
                                     "sm_mhz_median": clocks["sm_mhz"] if clocks else None,
                                     "hbm_floor_frac": (sw.bytes / (pass_ms * 1e-3) / 1e9) / peaks["hbm_gbs"]},
                     "kernels": {k: {"launches": v["launches"], "us": round(v["us"], 2), "share": round(v["share"], 4),
                                     "TFLOP/s": round(v["TFLOP/s"], 1),
                                     "dram_bytes_per_launch": SWEEP_DRAM_BYTES_PER_LAUNCH.get(k)}
                                 for k, v in sorted(groups.items(), key=lambda kv: -kv[1]["share"])}},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d_total, "d2h_bytes_per_step": d2h_total,
                "ms_per_step": e2e_s * 1e3, "step": "one pass over the work list",
                "host_gbs_per_gpu": (h2d_total + d2h_total) / world / e2e_s / 1e9},
        "gpu_launches": launches_per_pass * args.passes * args.steps,
        "clocks": clocks,
    }
    if replica is not None:
        line["replicas"] = replica
    if nsplit_row is not None:
        line["nsplit_gemm"] = nsplit_row
    if table is not None:
        del sw
        torch.cuda.empty_cache()
        line["roofline"]["configs"] = table
        line["extras"] = table_extras
        cores = host_threads()
        cpu = CpuSweep(cores)
        cpu.one_pass()
        dt = cpu.one_pass()
        line["cpu_baseline"] = {"value": cpu.flops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                                "gflops_per_core": cpu.flops / dt / 1e9 / cores, "sample": cpu.sample_text(dt)}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    global INSTANCES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["helix", "reference"], default="helix")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-configuration table and the CPU pass")
    ap.add_argument("--lanes", type=int, default=4, help="independent units run in this many concurrent chains per GPU")
    ap.add_argument("--passes", type=int, default=PASSES, help="passes over the work list per step")
    ap.add_argument("--instances", type=int, default=INSTANCES,
                    help="seeded copies of the sweep in the work list (default 8; 1 keeps a profiler run small)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    INSTANCES = max(1, args.instances)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        bench_reference(args, rank, world)
        return
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    bench_helix(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
