"""numpy front-end of the C oracle (``helix_oracle.c``).  Test infrastructure only.

Every function takes and returns numpy arrays; fp16 data travels as
``np.float16`` and is handed to C as raw 16-bit words.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libhelix_oracle.so")
_lib = None


def build(force=False):
    """Compile ``libhelix_oracle.so`` next to its source (gcc only)."""
    src = os.path.join(_HERE, "helix_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "libhelix_oracle.so"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_f32_to_f16.restype = None
        _lib.oracle_f16_to_f32.restype = None
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _chk(rc, what):
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


def max_threads():
    return int(lib().oracle_max_threads())


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _f16(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def sgemm_naive(a, b, fma=False):
    """C = A @ B as the reference's cpuSgemm loop (sgemm.cu:12-24)."""
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.empty((M, N), np.float32)
    _chk(lib().oracle_sgemm_naive(_p(a), _p(b), _p(c), M, N, K, int(fma)), "sgemm_naive")
    return c


def sgemm_f64acc(a, b):
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float32)
    _chk(lib().oracle_sgemm_f64acc(_p(a), _p(b), _p(c), M, N, K), "sgemm_f64acc")
    return c


def sgemm_template(a, b, m1, m2, n1, n2, k1, fma=False):
    """Single-thread x86 template loop nest (profile_x86_CPU.py:40-60)."""
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float32)
    _chk(lib().oracle_sgemm_template(_p(a), _p(b), _p(c), M, N, K, m1, m2, n1, n2, k1, int(fma)),
         "sgemm_template")
    return c


def sgemm_parallel(a, b, tiling=(8, 1, 32, 64, 1, 2, 6), threads=0, fma=False, out=None):
    """Parallel / packed op-level schedule (benchmark_x86_CPU_gemm.py:71-117).

    ``tiling`` = (m1, m2, m3, n1, n2, n3, k1) as returned by ``get_tiling``.
    """
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    _, N = b.shape
    c = np.empty((M, N), np.float32) if out is None else out
    m1, m2, m3, n1, n2, n3, k1 = tiling
    _chk(lib().oracle_sgemm_parallel(_p(a), _p(b), _p(c), M, N, K, m1, m2, m3, n1, n2, n3, k1,
                                     int(threads), int(fma)), "sgemm_parallel")
    return c


def gemv_f32_lane_tree(w, x):
    """y[m,rows] = x[m,K] . w[rows,K]^T in fp32, summed as a 32-lane streaming GEMV sums it (lane chains of
    fused multiply-adds over ascending k, then the xor tree); K a multiple of 4."""
    w, x = _f32(w), _f32(x)
    rows, K = w.shape
    m = x.shape[0]
    assert x.shape[1] == K
    y = np.empty((m, rows), np.float32)
    _chk(lib().oracle_gemv_f32_lane_tree(_p(w), _p(x), _p(y), rows, K, m), "gemv_f32_lane_tree")
    return y


def hgemm_naive(a, b, b_is_nk=True, fma=False):
    """fp16 x fp16 -> (fp16, fp32) as cpuF16F16Gemm (gemm.cu:26-37).

    ``b`` is N x K when ``b_is_nk`` (the layout the GPU kernels receive),
    else K x N as in the reference's host loop.
    """
    a, b = _f16(a), _f16(b)
    M, K = a.shape
    N = b.shape[0] if b_is_nk else b.shape[1]
    assert (b.shape[1] if b_is_nk else b.shape[0]) == K
    c16 = np.empty((M, N), np.float16)
    c32 = np.empty((M, N), np.float32)
    _chk(lib().oracle_hgemm_naive(_p(a), _p(b), _p(c16), _p(c32), M, N, K, int(b_is_nk), int(fma)),
         "hgemm_naive")
    return c16, c32


def hgemm_fast(a, b_nk, threads=0):
    """Blocked / vectorised fp16 GEMM (FP32 partial sums), for large shapes."""
    a, b = _f16(a), _f16(b_nk)
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K
    c16 = np.empty((M, N), np.float16)
    c32 = np.empty((M, N), np.float32)
    _chk(lib().oracle_hgemm_fast(_p(a), _p(b), _p(c16), _p(c32), M, N, K, int(threads)), "hgemm_fast")
    return c16, c32


def conv_out_hw(H, W, R, S, stride, pad):
    """Output extent, Ampere_FP16_conv.py:432."""
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


def conv2d_nhwc_f16(x, w, stride, pad):
    """x[N,H,W,C] * w[K,R,S,C] -> (y16, y32)[N,Ho,Wo,K], FP32 accumulate."""
    x, w = _f16(x), _f16(w)
    NB, H, W, C = x.shape
    KO, R, S, C2 = w.shape
    assert C == C2
    Ho, Wo = conv_out_hw(H, W, R, S, stride, pad)
    y16 = np.empty((NB, Ho, Wo, KO), np.float16)
    y32 = np.empty((NB, Ho, Wo, KO), np.float32)
    _chk(lib().oracle_conv2d_nhwc_f16(_p(x), _p(w), _p(y16), _p(y32), NB, H, W, C, KO, R, S, stride, pad),
         "conv2d_nhwc_f16")
    return y16, y32


def conv2d_nhwc_f32(x, w, stride, pad, fma=False):
    x, w = _f32(x), _f32(w)
    NB, H, W, C = x.shape
    KO, R, S, _ = w.shape
    Ho, Wo = conv_out_hw(H, W, R, S, stride, pad)
    y = np.empty((NB, Ho, Wo, KO), np.float32)
    _chk(lib().oracle_conv2d_nhwc_f32(_p(x), _p(w), _p(y), NB, H, W, C, KO, R, S, stride, pad, int(fma)),
         "conv2d_nhwc_f32")
    return y


def im2col_nchw_f32(im, ksize, stride, pad):
    """The reference's explicit im2col layout (im2col.cu:37-75)."""
    im = _f32(im)
    NB, C, H, W = im.shape
    Ho, Wo = conv_out_hw(H, W, ksize, ksize, stride, pad)
    col = np.empty((NB, C * ksize * ksize, Ho, Wo), np.float32)
    _chk(lib().oracle_im2col_nchw_f32(_p(im), _p(col), NB, C, H, W, ksize, stride, pad), "im2col")
    return col


def f32_to_f16(a):
    a = _f32(a)
    out = np.empty(a.shape, np.float16)
    lib().oracle_f32_to_f16(_p(a), _p(out), ctypes.c_size_t(a.size))
    return out


def f16_to_f32(a):
    a = _f16(a)
    out = np.empty(a.shape, np.float32)
    lib().oracle_f16_to_f32(_p(a), _p(out), ctypes.c_size_t(a.size))
    return out
