#!/usr/bin/env python
"""Benchmark of the Helix hot path on B200: the model-level fp16 GEMM / convolution sweep.

One step = one pass over the model-level sweep (every GEMM of a BERT-base encoder at batch 16,
seq 512 plus the 53 ResNet-50 convolutions at batch 32, 125 independent units, 1.81 TFLOP).
Each rank runs the whole sweep on its own GPU with its own data (weak scaling, no collective
in the data path).  Prints ONE JSON line (rank 0).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl helix|reference]

`--impl reference` times the CPU restatement of the reference's x86 template (the reference's
own CPU path is TVM generated and cannot be built here) on a bounded sample of the same sweep.
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
WORKLOAD = "model-level sweep: BERT-base b16 s512 (72 GEMMs incl. batched QK^T/PV) + ResNet-50 b32 224x224 (53 convs)"


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the x86 template on a bounded sample of the sweep
# ----------------------------------------------------------------------------------------------
def cpu_sample_units():
    """One BERT layer's four linear GEMMs, 8 of its 192 batched attention GEMMs of each kind,
    and three ResNet-50 convolutions as GEMMs (M = B*Ho*Wo, N = OC, K = IC*kH*kW, batch 4)."""
    return [
        ("bert.qkv", (8192, 2304, 768), 1), ("bert.out_proj", (8192, 768, 768), 1),
        ("bert.ffn_up", (8192, 3072, 768), 1), ("bert.ffn_down", (8192, 768, 3072), 1),
        ("bert.qk", (512, 512, 64), 8), ("bert.pv", (512, 64, 512), 8),
        ("resnet.s1.conv2", (4 * 56 * 56, 64, 576), 1), ("resnet.s3.conv2", (4 * 14 * 14, 256, 2304), 1),
        ("resnet.s4.conv3", (4 * 7 * 7, 2048, 512), 1),
    ]


def run_cpu_sample(min_seconds=10.0):
    """Seconds per pass, flops per pass, threads and passes of the sample with all host threads (fp32, as
    the reference's x86 backend computes); whole passes are repeated until `min_seconds` have gone by."""
    import numpy as np
    from oracle import api
    units = cpu_sample_units()
    rng = np.random.default_rng(4)
    mats = []
    for _, (M, N, K), cnt in units:
        s = np.float32(1.0 / np.sqrt(K))
        a = (rng.standard_normal((M, K), dtype=np.float32) * s)
        b = (rng.standard_normal((K, N), dtype=np.float32) * s)
        mats.append((a, b, np.empty((M, N), np.float32), cnt))
    flops = sum(2.0 * M * N * K * cnt for _, (M, N, K), cnt in units)
    api.sgemm_parallel(mats[1][0], mats[1][1], out=mats[1][2])  # warm the thread pool
    passes = 0
    t0 = time.perf_counter()
    while True:
        for a, b, c, cnt in mats:
            for _ in range(cnt):
                api.sgemm_parallel(a, b, out=c)
        passes += 1
        if time.perf_counter() - t0 >= min_seconds:
            break
    dt = (time.perf_counter() - t0) / passes
    return dt, flops, api.max_threads(), passes


def bench_reference(args, rank, world):
    if rank != 0:
        return
    times = []
    flops = cores = passes = None
    for i in range(args.warmup + args.steps):
        dt, flops, cores, passes = run_cpu_sample()
        if i >= args.warmup:
            times.append(dt)
    avg = sum(times) / len(times)
    value = flops / avg / 1e12
    sample = ("one BERT-base layer (4 linear GEMMs + 8 of 192 QK^T and PV GEMMs) and 3 ResNet-50 convs as "
              "GEMMs at batch 4, fp32, %.1f GFLOP per pass, %d passes (>= 10 s) per step" % (flops / 1e9, passes))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": avg * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "bounded CPU sample of the sweep; a step repeats the sample pass for >= 10 s and ms_per_step "
                                                  "is the time of one pass; throughput extrapolates"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
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
        sm, reasons, mx = [], set(), None
        try:
            with open(self.path) as f:
                for line in f:
                    p = [x.strip() for x in line.split(",")]
                    if len(p) < 9:
                        continue
                    try:
                        sm.append(float(p[1]))
                        mx = float(p[2])
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
            sm.sort()
            # the busy half of the samples: the sampler also sees the idle edges of the region
            busy = sm[len(sm) // 2:]
            out["sm_mhz"] = busy[len(busy) // 2]
            out["sm_max_mhz"] = mx
            out["sm_min_mhz_seen"] = sm[0]
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def extras(peaks):
    """Per-configuration figures beside the headline: GEMV GB/s, dense GEMM sweep, convs, fp32 GEMM."""
    import torch
    from helix_b200 import datagen, ops
    from helix_b200._lib import LAUNCH_INDEPENDENT, LAUNCH_STATIC_A
    out = {}
    dev = "cuda"
    # fp16 GEMV 4096 x 4096, m = 1: rotating W buffers (12 x 32 MiB > 2 x L2), CUDA-graph timing
    rows = K = 4096
    ws = [torch.randn(rows, K, device=dev, dtype=torch.float16) * 0.02 for _ in range(12)]
    x = torch.randn(1, K, device=dev, dtype=torch.float16)
    ys = [torch.empty(1, rows, device=dev, dtype=torch.float16) for _ in ws]
    ls = [ops.launch_gemv_f16(w, x, y) for w, y in zip(ws, ys)]
    gemv_bytes = rows * K * 2 + K * 2 + rows * 2
    res = {}
    # twelve distinct W / y pairs sharing only the read-only x: consecutive launches are independent.
    # Also reported: weights-static ordering (X may come from the previous kernel) and full ordering.
    for name, flag in (("independent", LAUNCH_INDEPENDENT), ("static_weights", LAUNCH_STATIC_A), ("ordered", 0)):
        for l in ls:
            l.flags = flag
        avg, _, _ = ops.time_launches(ls, warmup=5, iters=50, use_graph=True)
        gb = gemv_bytes / avg / 1e9
        res[name] = {"us": avg * 1e6, "GB/s": gb, "frac_hbm_peak": gb / peaks["hbm_gbs"]}
    out["gemv_4096x4096_m1"] = dict(res["independent"], launch_ordering=res)
    del ws, ys, ls
    # fp16 dense GEMM sweep
    gem = {}
    for (M, N, K) in datagen.C3_SHAPES:
        by = 2.0 * (M * K + N * K + M * N)
        nbuf = 1 if (2.0 * M * N * K / by) > 300 else int(300e6 // by) + 1
        bufs = [(torch.randn(M, K, device=dev, dtype=torch.float16) / K ** 0.5,
                 torch.randn(N, K, device=dev, dtype=torch.float16) / K ** 0.5,
                 torch.empty(M, N, device=dev, dtype=torch.float16)) for _ in range(nbuf)]
        ls = [ops.launch_gemm_f16(a, b, c) for a, b, c in bufs]
        if len(ls) > 1:
            for l in ls:
                l.flags = LAUNCH_INDEPENDENT
        avg, _, _ = ops.time_launches(ls, warmup=3, iters=20, use_graph=True)
        tf = 2.0 * M * N * K / avg / 1e12
        gem[f"{M}x{N}x{K}"] = {"us": avg * 1e6, "TFLOP/s": tf, "frac_tensor_peak": tf / peaks["tflops"],
                               "GB/s": by / avg / 1e9, "frac_hbm_peak": by / avg / 1e9 / peaks["hbm_gbs"]}
        del bufs, ls
    out["gemm_f16"] = gem
    # ResNet-style convolutions at batch 32
    conv = {}
    for layer in datagen.C4_LAYERS:
        B, C, H, W, OC, kh, kw, s, p = layer
        xx = torch.rand(B, H, W, C, device=dev, dtype=torch.float16) * 2 - 1
        ww = torch.randn(OC, kh, kw, C, device=dev, dtype=torch.float16) * (2.0 / (C * kh * kw)) ** 0.5
        Ho, Wo = ops.conv_out_hw(H, W, kh, kw, s, p)
        yy = torch.empty(B, Ho, Wo, OC, device=dev, dtype=torch.float16)
        l = ops.launch_conv2d_f16(xx, ww, yy, s, p)
        avg, _, _ = ops.time_launches([l] * 4, warmup=3, iters=20, use_graph=True)
        fl = 2.0 * B * Ho * Wo * OC * C * kh * kw
        by = 2.0 * (xx.numel() + ww.numel() + yy.numel())
        conv["x".join(map(str, layer))] = {"us": avg * 1e6, "TFLOP/s": fl / avg / 1e12,
                                          "frac_tensor_peak": fl / avg / 1e12 / peaks["tflops"],
                                          "GB/s": by / avg / 1e9}
    out["conv_f16"] = conv
    # fp32 FFMA GEMM: 1024^3 is the configuration the reference's CPU template runs; the larger squares show
    # the kernel with the machine full.  Rated against the nominal FFMA peak and against the rate a
    # register-resident FFMA stream of the same 8x8 block pattern reaches on this device.
    ffma_measured = ops.probe_ffma_f32()
    out["ffma_probe_tflops"] = ffma_measured
    for n in (1024, 2048, 4096):
        a = torch.rand(n, n, device=dev) * 2 - 1
        b = torch.rand(n, n, device=dev) * 2 - 1
        c = torch.empty(n, n, device=dev)
        avg, _, _ = ops.time_launches([ops.launch_gemm_f32(a, b, c)] * 4, warmup=3, iters=10, use_graph=True)
        tf = 2.0 * n ** 3 / avg / 1e12
        out["gemm_f32_%d" % n] = {"us": avg * 1e6, "TFLOP/s": tf, "frac_ffma_peak_nominal_74.4": tf / 74.4,
                                  "frac_ffma_probe": tf / ffma_measured}
        del a, b, c
    # true-fp32 convolution (column matrix + weight transpose + FFMA GEMM, all three kernels timed)
    from helix_b200 import harness
    c32 = {}
    for layer in datagen.C4_LAYERS[:2] + datagen.C4_LAYERS[3:4]:
        B, C, H, W, OC, kh, kw, s, p = layer
        t = harness.time_conv_f32(*layer)
        Ho, Wo = ops.conv_out_hw(H, W, kh, kw, s, p)
        tf = 2.0 * B * Ho * Wo * OC * C * kh * kw / t / 1e12
        c32["x".join(map(str, layer))] = {"us": t * 1e6, "TFLOP/s": tf, "frac_ffma_peak_nominal_74.4": tf / 74.4,
                                          "frac_ffma_probe": tf / ffma_measured}
    out["conv_f32"] = c32
    return out


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum, averaged over the launches of
# one sweep step) for each kernel of the sweep, from one single-pass ncu capture of
#   python bench.py --steps 1 --warmup 3 --no-extras
# Filled in below only for the kernels that capture listed; the others report null.
SWEEP_DRAM_BYTES_PER_LAUNCH = {
    "gemm_f16_tc2_kernel<256>": 15810162, "gemm_f16_tc2_kernel<192>": 34526677,
    "gemm_f16_tc_kernel<256,0>": 30764491, "gemm_f16_tc_kernel<64,0>": 68126530,
    "gemm_f16_tc_kernel<128,0>": 14688633, "gemm_f16_tc_kernel<64,1>": 26433792,
}


def kernel_breakdown(sw, ops):
    """Time the sweep's launches grouped by the kernel they resolve to (CUDA-graph replay, events on the
    launching stream): launches, seconds and algorithmic flop / bytes per group."""
    from helix_b200 import workloads
    import ctypes
    from helix_b200._lib import Launch
    groups = {}
    for u, l0 in zip(sw.units, sw.launches):
        # each kernel is rated on the whole machine, whatever share of it the sweep's lanes give a launch
        l = Launch()
        ctypes.memmove(ctypes.byref(l), ctypes.byref(l0), ctypes.sizeof(Launch))
        ops.limit_ctas(l, 0)
        g = groups.setdefault(ops.kernel_name(l), {"launches": [], "flop": 0.0, "bytes": 0.0})
        g["launches"].append(l)
        g["flop"] += workloads.unit_flops(u)
        g["bytes"] += workloads.unit_bytes(u)
    out = {}
    for name, g in groups.items():
        avg, _, _ = ops.time_launches(g["launches"], warmup=3, iters=10, use_graph=True)
        n = len(g["launches"])
        out[name] = {"launches": n, "us": avg * n * 1e6, "flop": g["flop"], "bytes": g["bytes"]}
    total = sum(v["us"] for v in out.values())
    for v in out.values():
        v["share"] = v["us"] / total
        v["TFLOP/s"] = v["flop"] / (v["us"] * 1e-6) / 1e12
    return out


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
    # one rank per GPU: keep this rank's pinned host buffers on its GPU's NUMA node (matters for e2e at N > 1)
    numa_cpus = dist_util.bind_to_gpu_numa_node(local_rank) if world > 1 else None

    units = workloads.model_level_sweep()
    sw = sweep.Sweep(units, seed=4 * 1000 + rank, lanes=args.lanes)
    # warm-up outside any capture: sets function attributes, fills the tensor-map cache
    launches_per_step = sw.step()
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

    def one_step():
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
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        one_step()
    e1.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    ops.check_status()
    ms = dist_util.max_over_ranks(ms, dist, "cuda")
    ms_per_step = ms / args.steps
    value = sw.flops * world / (ms_per_step * 1e-3) / 1e12

    # end to end: pinned host operands in, results out, every step
    hs = sweep.HostSweep(sw)
    e2e_steps = max(1, min(args.steps, 3))
    hs.step()
    hs.finish()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        hs.step()
    hs.finish()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = dist_util.max_over_ranks(e2e_s, dist, "cuda")
    e2e_value = sw.flops * world / e2e_s / 1e12
    ops.check_status()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    peak = peaks["tflops_sustained"]
    per_gpu = value / world
    # dominant kernel: the group with the largest share of the step's device time
    groups = kernel_breakdown(sw, ops)
    ops.check_status()
    top = max(groups, key=lambda k: groups[k]["share"])
    tg = groups[top]
    traffic = SWEEP_DRAM_BYTES_PER_LAUNCH.get(top)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 in / f32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "units_per_step_per_gpu": len(units), "flop_per_step_per_gpu": sw.flops,
                   "cache": "operands of one step total %.1f GB per GPU (> L2), one buffer set per unit" % (sw.bytes / 1e9),
                   "cuda_graph": graph is not None, "parallelism": f"independent replicas of the sweep x{world}",
                   "lanes": "%d concurrent launch chains per GPU, each launch limited to 1/%d of the SMs" % (args.lanes, args.lanes),
                   "host_numa_binding": ("rank 0 bound to %d CPUs next to its GPU" % len(numa_cpus)) if numa_cpus else "none"},
        "roofline": {"bound": "tensor", "achieved": tg["TFLOP/s"], "peak": peak, "unit": "TFLOP/s",
                     "frac": tg["TFLOP/s"] / peak, "traffic": traffic,
                     "kernel": top, "launches_per_step": tg["launches"], "share_of_step": tg["share"],
                     "us_per_launch": tg["us"] / tg["launches"],
                     "algorithmic_flop_per_launch": tg["flop"] / tg["launches"],
                     "algorithmic_bytes_per_launch": tg["bytes"] / tg["launches"],
                     "peak_source": peaks["source"] + " (sustained bf16 cuBLAS; burst %.0f)" % peaks["tflops"],
                     "whole_sweep": {"achieved": per_gpu, "frac": per_gpu / peak,
                                     "hbm_floor_frac": (sw.bytes / (ms_per_step * 1e-3) / 1e9) / peaks["hbm_gbs"]},
                     "kernels": {k: {"launches": v["launches"], "us": round(v["us"], 2), "share": round(v["share"], 4),
                                     "TFLOP/s": round(v["TFLOP/s"], 1),
                                     "dram_bytes_per_launch": SWEEP_DRAM_BYTES_PER_LAUNCH.get(k)}
                                 for k, v in sorted(groups.items(), key=lambda kv: -kv[1]["share"])}},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": hs.h2d_bytes * world,
                "d2h_bytes_per_step": hs.d2h_bytes * world, "ms_per_step": e2e_s * 1e3},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    if world == 1 and not args.no_extras:
        del hs
        torch.cuda.empty_cache()
        # the per-shape table runs on a GPU the sweep has already heated: record the clocks it saw
        xs = ClockSampler(local_rank)
        xs.start()
        line["extras"] = extras(peaks)
        line["extras"]["clocks"] = xs.stop()
        dt, flops, cores, passes = run_cpu_sample()
        line["cpu_baseline"] = {
            "value": flops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": "one BERT-base layer (4 linear GEMMs + 8 of 192 QK^T and PV GEMMs) and 3 ResNet-50 convs as GEMMs "
                      "at batch 4, fp32 x86-template restatement, %d passes of %.1f GFLOP in %.1f s"
                      % (passes, flops / 1e9, dt * passes)}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["helix", "reference"], default="helix")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-configuration table and CPU sample")
    ap.add_argument("--lanes", type=int, default=2, help="independent shapes of the sweep run in this many concurrent chains")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
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
