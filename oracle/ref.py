"""ctypes access to the reference's own host loops compiled into ``oracle/_ref``.

``make -C oracle ref`` compiles the unmodified reference files
``src_template/Ampere_FP32/sgemm.cu`` and ``src_template/Ampere_FP16/gemm.cu``
into shared objects; this module calls only their host functions ``cpuSgemm``
(sgemm.cu:12-24) and ``cpuF16F16Gemm`` (gemm.cu:26-37).  Test infrastructure
only; available wherever the prebuilt ``_ref`` directory is present.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_REF_DIR = os.path.join(_HERE, "_ref")
_SGEMM_SO = os.path.join(_REF_DIR, "libref_sgemm.so")
_HGEMM_SO = os.path.join(_REF_DIR, "libref_hgemm.so")


def _find_reference_tree():
    """The reference checkout: HELIX_REFERENCE_TREE, else a directory named ``reference`` beside this
    repository; an empty string when neither holds the reference's src_template/."""
    repo = os.path.dirname(_HERE)
    for cand in (os.environ.get("HELIX_REFERENCE_TREE", ""), os.path.join(os.path.dirname(repo), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src_template")):
            return cand
    return ""


REFERENCE_TREE = _find_reference_tree()


def build():
    """Build ``oracle/_ref`` if the reference tree is present; returns availability."""
    if available():
        return True
    if not REFERENCE_TREE:
        return False
    subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REF={REFERENCE_TREE}"])
    return available()


def available():
    return os.path.exists(_SGEMM_SO) and os.path.exists(_HGEMM_SO)


_libs = {}


def _load(path):
    if path not in _libs:
        _libs[path] = ctypes.CDLL(path)
    return _libs[path]


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def cpuSgemm(a, b):
    """The reference's FP32 host loop: a[M,K] @ b[K,N] -> c[M,N]."""
    a = np.ascontiguousarray(a, np.float32)
    b = np.ascontiguousarray(b, np.float32)
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float32)
    fn = _load(_SGEMM_SO)._Z8cpuSgemmPfS_S_iii
    fn.restype = None
    fn(_p(a), _p(b), _p(c), M, N, K)
    return c


def cpuF16F16Gemm(a, b_kn):
    """The reference's fp16 host loop: a[M,K] @ b[K,N] -> c[M,N] (fp16)."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b_kn)
    assert a.dtype == np.float16 and b.dtype == np.float16
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float16)
    fn = _load(_HGEMM_SO)._Z13cpuF16F16GemmP6__halfS0_S0_iii
    fn.restype = None
    fn(_p(a), _p(b), _p(c), M, N, K)
    return c
