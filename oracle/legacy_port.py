"""Context rows: the reference's own Ampere kernels, unmodified, recompiled for sm_100a and run on this GPU
the way the reference drives them.

`make -C oracle legacy REF=<reference checkout>` builds a subset of the reference's executables into
``oracle/_ref/legacy`` (the built files travel with the repository snapshot).  This script then

  1. profiles every built fp16 configuration with the reference's own probe -- one CTA's problem
     ``M = BLOCK_ROWS, N = BLOCK_COLS, K = 4096``, the GEMVs at ``1 128 1024`` -- into a dictionary keyed
     ``(K_STAGE, BR, BC, WR, WC, splitK)`` (scripts/Ampere_FP16/profile_Ampere_FP16.py:17-62);
  2. picks a configuration per shape with the reference's cost model, ``ceil(tiles * (splitK + 1) / 108) * t_cfg``
     (scripts/Ampere_FP16/Ampere_FP16_gemm.py:420-430; the literal 108 is the reference's), and runs it on the
     shape padded to tile multiples (``:432-441``);
  3. runs convolutions as the reference does: its NCHW ``im2col`` executable followed by the picked GEMM at
     ``M = B*Ho*Wo, N = OC, K = IC*kH*kW`` (scripts/Ampere_FP16/Ampere_FP16_conv.py:431-446), the two times added;
  4. also reports the best configuration of the built subset per shape (what an exhaustive search over the
     subset would get), and the fp32 and GEMV executables.

Each executable allocates uninitialised buffers, runs 10 warm-up and 10 timed launches and prints one line whose
whitespace token [-8] is the average time in seconds (src_template/Ampere_FP16/gemm.cu:687-689; the gemv line
labels it "ms" but divides its millisecond figure by 1e3 first, gemv.cu:394-399).  The reference's ``im2col``
executable prints its average microseconds divided by 1e9 with "%f" (im2col.cu:191), i.e. 0.000000, so its time
comes from ``im2col_us``: the same unmodified source and timing routine behind an entry point that prints the
microseconds (oracle/legacy_im2col_main.cu).  Measurement context only: nothing in the library, the tests
or bench.py uses it.

  python oracle/legacy_port.py [--json out.json] [--only gemm|conv|other]
"""
import argparse
import json
import math
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LEGACY = os.path.join(HERE, "_ref", "legacy")

HGEMM_SHAPES = [(4096, 4096, 4096), (8192, 8192, 8192), (16, 11008, 4096), (128, 4096, 11008), (2048, 14336, 4096)]
SGEMM_SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096)]
GEMV_SHAPES = [(1, 4096, 4096), (1, 16384, 8192)]
# (batch, IC, H, W, OC, kH, kW, stride, pad): the five ResNet-style layers at batch 32
CONV_LAYERS = [(32, 64, 56, 56, 64, 3, 3, 1, 1), (32, 128, 28, 28, 128, 3, 3, 1, 1), (32, 256, 14, 14, 256, 3, 3, 1, 1),
               (32, 256, 56, 56, 64, 1, 1, 1, 0), (32, 128, 56, 56, 128, 3, 3, 2, 1)]
REFERENCE_SM_COUNT = 108   # the literal in the reference's cost model (an A100)


def run_exe(path, *ints, timeout=300):
    """Average seconds reported by one reference GEMM / GEMV executable, or None if it printed no result line."""
    try:
        out = subprocess.run([path] + [str(v) for v in ints], capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return None
    for line in reversed(out.stdout.splitlines()):
        tok = line.split()
        if line.startswith("M N K =") and len(tok) >= 8:
            try:
                return float(tok[-8])
            except ValueError:
                return None
    return None


def run_im2col(path, layer, timeout=300):
    """Microseconds per launch of the reference's im2col kernel for one layer (im2col_us), or None."""
    try:
        out = subprocess.run([path] + [str(v) for v in layer], capture_output=True, text=True, timeout=timeout)
        return float(out.stdout.split()[0])
    except (subprocess.TimeoutExpired, ValueError, IndexError):
        return None


def exe_key(name):
    """'gemm_4_128_256_64_64' -> (4, 128, 256, 64, 64, 0); 'gemm_splitK_...' -> (..., 1); the GEMVs as the
    reference keys them; None for anything else."""
    if name == "gemv":
        return (0, 1, 128, 0, 0, 0)
    if name == "gemv_splitK":
        return (0, 1, 128, 0, 0, 1)
    for prefix, sk in (("gemm_splitK_", 1), ("gemm_", 0)):
        if name.startswith(prefix):
            try:
                f = tuple(int(v) for v in name[len(prefix):].split("_"))
            except ValueError:
                return None
            return f + (sk,) if len(f) == 5 else None
    return None


def exe_name(key):
    if key[0] == 0:
        return "gemv" if key[5] == 0 else "gemv_splitK"
    return ("gemm_" if key[5] == 0 else "gemm_splitK_") + "_".join(str(v) for v in key[:5])


def profile(exes):
    """The reference's profile over the built subset: seconds of each configuration on its one-CTA probe."""
    prof = {}
    for e in exes:
        key = exe_key(e)
        if key is None:
            continue
        t = run_exe(os.path.join(LEGACY, e), 1, 128, 1024) if key[0] == 0 else \
            run_exe(os.path.join(LEGACY, e), key[1], key[2], 4096)
        if t is not None and t > 0:
            prof[key] = t
    return prof


def reference_cost_model(prof, M, N, K, sms=REFERENCE_SM_COUNT):
    """argmin over the dictionary of waves x probe time; K plays no part, as in the reference."""
    best, best_cost = None, float("inf")
    for key, t in prof.items():
        blocks = math.ceil(M / key[1]) * math.ceil(N / key[2]) * (key[5] + 1)
        cost = math.ceil(blocks / sms) * t
        if cost < best_cost:
            best, best_cost = key, cost
    return best


def run_config(key, M, N, K):
    """Seconds of one configuration on (M, N, K), launched as the reference launches it."""
    path = os.path.join(LEGACY, exe_name(key))
    if key[0] == 0:
        return run_exe(path, M, N, K)
    return run_exe(path, math.ceil(M / key[1]) * key[1], math.ceil(N / key[2]) * key[2], K)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--only", choices=["all", "gemm", "conv", "other"], default="all",
                    help="run one group of rows (the profile always runs: the pick needs it)")
    args = ap.parse_args(argv)
    if not os.path.isdir(LEGACY):
        print("oracle/_ref/legacy is missing: run `make -C oracle legacy REF=<reference checkout>`")
        return 1
    exes = sorted(os.listdir(LEGACY))
    rows = []
    prof = profile(exes)
    print("profiled %d fp16 configurations (one-CTA probe, seconds):" % len(prof))
    for key in sorted(prof):
        print("  %-28s %.3e" % (exe_name(key), prof[key]), flush=True)

    def bytes_of(M, N, K, e=2.0):
        return e * (M * K + N * K + M * N)

    # fp16 GEMMs: the reference's pick, and the best of the subset
    gemm_keys = [k for k in prof if k[0] != 0]
    for (M, N, K) in (HGEMM_SHAPES if args.only in ("all", "gemm") else []):
        pick = reference_cost_model(prof, M, N, K)
        t_pick = run_config(pick, M, N, K) if pick else None
        best = None
        for key in gemm_keys:
            t = run_config(key, M, N, K)
            if t and t > 0 and (best is None or t < best[1]):
                best = (key, t)
        row = {"kind": "gemm_f16", "shape": [M, N, K]}
        if t_pick:
            row.update({"cost_model_pick": exe_name(pick), "pick_us": t_pick * 1e6,
                        "pick_TFLOP/s": 2.0 * M * N * K / t_pick / 1e12, "pick_GB/s": bytes_of(M, N, K) / t_pick / 1e9})
        if best:
            row.update({"best_of_subset": exe_name(best[0]), "best_us": best[1] * 1e6,
                        "best_TFLOP/s": 2.0 * M * N * K / best[1] / 1e12, "best_GB/s": bytes_of(M, N, K) / best[1] / 1e9})
        print(json.dumps(row), flush=True)
        rows.append(row)

    # convolutions: im2col executable + the picked GEMM, the reference's two-process path
    im2col = os.path.join(LEGACY, "im2col_us")
    if os.path.exists(im2col) and args.only in ("all", "conv"):
        for layer in CONV_LAYERS:
            B, IC, H, W, OC, kH, kW, stride, pad = layer
            M = B * ((H + 2 * pad - kH) // stride + 1) * ((W + 2 * pad - kW) // stride + 1)
            N, K = OC, IC * kH * kW
            pick = reference_cost_model(prof, M, N, K)
            t_col = run_im2col(im2col, layer)
            t_gemm = run_config(pick, M, N, K) if pick else None
            best = None
            for key in gemm_keys:
                t = run_config(key, M, N, K)
                if t and t > 0 and (best is None or t < best[1]):
                    best = (key, t)
            row = {"kind": "conv_f16 (im2col + gemm)", "layer": list(layer), "gemm": [M, N, K], "im2col_us": t_col}
            if t_gemm and t_col:
                tot = t_col + t_gemm * 1e6
                row.update({"cost_model_pick": exe_name(pick), "pick_gemm_us": t_gemm * 1e6, "pick_total_us": tot,
                            "pick_TFLOP/s": 2.0 * M * N * K / tot / 1e6})
            if best and t_col:
                tot = t_col + best[1] * 1e6
                row.update({"best_of_subset": exe_name(best[0]), "best_gemm_us": best[1] * 1e6, "best_total_us": tot,
                            "best_TFLOP/s": 2.0 * M * N * K / tot / 1e6})
            print(json.dumps(row), flush=True)
            rows.append(row)

    # fp32 GEMM and GEMV executables: best of the built ones
    for prefix, shapes in ((("sgemm_", SGEMM_SHAPES), ("gemv", GEMV_SHAPES)) if args.only in ("all", "other") else ()):
        for (M, N, K) in shapes:
            best = None
            for e in exes:
                if not e.startswith(prefix):
                    continue
                t = run_exe(os.path.join(LEGACY, e), M, N, K)
                if t is None or t <= 0:
                    continue
                if best is None or t < best[1]:
                    best = (e, t)
            if best:
                row = {"kind": prefix.rstrip("_"), "shape": [M, N, K], "best": best[0], "us": best[1] * 1e6,
                       "TFLOP/s": 2.0 * M * N * K / best[1] / 1e12,
                       "GB/s": bytes_of(M, N, K, 4.0 if prefix == "sgemm_" else 2.0) / best[1] / 1e9}
                print(json.dumps(row), flush=True)
                rows.append(row)
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"profile": {exe_name(k): v for k, v in prof.items()}, "rows": rows}, f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
