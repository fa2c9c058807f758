"""In-tree build of ``libhelix_b200.so`` (nvcc, sm_100a only).

Stands in for the reference's generator loop, which runs nvcc once per tile
configuration and leaves one executable per configuration in ``build/bin_fp16``
/ ``build/bin_fp32`` (scripts/Ampere_FP16/build_Ampere_FP16.py:41-70,
scripts/Ampere_FP32/build_Ampere_FP32.py:37-63).  Here every configuration is a
template instantiation inside one shared library; translation units compile in
parallel and are skipped when their sources have not changed.
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(CSRC, "_obj")
LIB_PATH = os.path.join(PKG_DIR, "libhelix_b200.so")
SOURCES = ["capi.cu", "gemv_f16.cu", "sgemm_f32.cu", "gemm_f16_tc.cu", "gemm_f16_tc2.cu", "conv_f16_halo.cu", "conv_f16_stem.cu", "conv_f16_rows.cu", "conv_f32.cu", "gemv_f32.cu"]
HEADERS = ["common.cuh", "conv_common.cuh", "kernels.h", os.path.join("..", "..", "include", "helix_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _compile_one(src, verbose):
    src_path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    stamp = obj + ".sha"
    dig = _digest([src_path] + [os.path.join(CSRC, h) for h in HEADERS], " ".join(NVCC_FLAGS))
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
        return obj, False, ""
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src_path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    with open(stamp, "w") as f:
        f.write(dig)
    return obj, True, res.stderr


def build(verbose=False, force=False):
    """Compile (if stale) and link the library; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            os.remove(os.path.join(OBJ_DIR, f))
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda s: _compile_one(s, verbose), SOURCES))
    objs = [r[0] for r in results]
    rebuilt = any(r[1] for r in results)
    if verbose:
        for r in results:
            if r[2]:
                sys.stderr.write(r[2])
    if rebuilt or not os.path.exists(LIB_PATH):
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB_PATH] + objs
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
