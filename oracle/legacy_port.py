"""Context rows: the reference's own Ampere kernels, unmodified, recompiled for sm_100a and run on this GPU.

`make -C oracle legacy` builds a few of the reference's executables into ``oracle/_ref/legacy``
(needs the reference tree; the built files travel with the repository snapshot).  This script
runs them on the benchmark shapes with the reference's own protocol -- each executable allocates
uninitialised buffers, runs 10 warm-up and 10 timed launches and prints one line whose
whitespace token [-8] is the average time in seconds (scripts/Ampere_FP16/Ampere_FP16_gemm.py:432-441,
src_template/Ampere_FP16/gemm.cu:687-689; the gemv line labels it "ms" but divides its millisecond
figure by 1e3 first, gemv.cu:394-399) -- and prints the best configuration per shape.  Measurement context only:
nothing in the library, the tests or bench.py uses it.

  python oracle/legacy_port.py [--json out.json]
"""
import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LEGACY = os.path.join(HERE, "_ref", "legacy")

HGEMM_SHAPES = [(4096, 4096, 4096), (8192, 8192, 8192), (2048, 14336, 4096)]
SGEMM_SHAPES = [(1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096)]
GEMV_SHAPES = [(1, 4096, 4096), (1, 16384, 8192)]


def run_exe(path, M, N, K, timeout=300):
    """Average seconds reported by one reference executable, or None if it printed no result line."""
    out = subprocess.run([path, str(M), str(N), str(K)], capture_output=True, text=True, timeout=timeout)
    for line in reversed(out.stdout.splitlines()):
        tok = line.split()
        if line.startswith("M N K =") and len(tok) >= 8:
            return float(tok[-8])
    return None


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)
    if not os.path.isdir(LEGACY):
        print("oracle/_ref/legacy is missing: run `make -C oracle legacy` where the reference tree is present")
        return 1
    exes = sorted(os.listdir(LEGACY))
    rows = []
    for prefix, shapes in (("gemm_", HGEMM_SHAPES), ("sgemm_", SGEMM_SHAPES), ("gemv", GEMV_SHAPES)):
        for (M, N, K) in shapes:
            best = None
            for e in exes:
                if not e.startswith(prefix) or (prefix == "gemm_" and e.startswith("gemv")):
                    continue
                t = run_exe(os.path.join(LEGACY, e), M, N, K)
                if t is None or t <= 0:
                    continue
                tf = 2.0 * M * N * K / t / 1e12
                print(f"{e:32s} {M}x{N}x{K}: {t * 1e6:10.1f} us {tf:9.2f} TFLOP/s", flush=True)
                if best is None or t < best[1]:
                    best = (e, t)
            if best:
                rows.append({"kind": prefix.rstrip("_"), "shape": [M, N, K], "best": best[0], "us": best[1] * 1e6,
                             "TFLOP/s": 2.0 * M * N * K / best[1] / 1e12,
                             "GB/s": 2.0 * (M * K + N * K + M * N) / best[1] / 1e9 if prefix != "sgemm_" else
                             4.0 * (M * K + N * K + M * N) / best[1] / 1e9})
    print(json.dumps(rows))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f)
    return 0


if __name__ == "__main__":
    sys.exit(main())
