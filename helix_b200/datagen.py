"""Seeded synthetic inputs for the five benchmark configurations.

All tensors are drawn on the host with ``numpy.random.default_rng(seed)`` in a
fixed order (first the activation-like operand, then the weight-like one) and
cast once, so the CPU oracle and the GPU kernels see identical bytes whichever
device a shape is scheduled on.  The shape suites stand in for the reference's
shape lists (scripts/utils/get_benchmark_shape_list.py) with random data: the
reference itself times uninitialised buffers (src_template/Ampere_FP16/gemm.cu
:632-634), so no dataset content is involved.
"""
import numpy as np

# (M, N, K) of the FP16 dense-GEMM sweep.
C3_SHAPES = [(4096, 4096, 4096), (8192, 8192, 8192), (16, 11008, 4096),
             (128, 4096, 11008), (2048, 14336, 4096)]

# (batch, IC, H, W, OC, kH, kW, stride, pad): same tuple order as the reference's
# conv shape lists (scripts/Ampere_FP16/benchmark_Ampere_FP16_conv.py:15).
C4_LAYERS = [
    (32, 64, 56, 56, 64, 3, 3, 1, 1),
    (32, 128, 28, 28, 128, 3, 3, 1, 1),
    (32, 256, 14, 14, 256, 3, 3, 1, 1),
    (32, 256, 56, 56, 64, 1, 1, 1, 0),
    (32, 128, 56, 56, 128, 3, 3, 2, 1),
]


def shape_seed(base_seed, index):
    """Seed of the ``index``-th unit of a sweep: independent of the GPU it runs on."""
    return int(np.random.SeedSequence([int(base_seed), int(index)]).generate_state(1)[0])


def c1_fp32_gemm(M=1024, N=1024, K=1024, seed=0):
    """A[M,K], B[K,N] float32 i.i.d. U[-1,1]."""
    rng = np.random.default_rng(seed)
    a = rng.uniform(-1.0, 1.0, (M, K)).astype(np.float32)
    b = rng.uniform(-1.0, 1.0, (K, N)).astype(np.float32)
    return a, b


def c2_gemv(rows=4096, K=4096, m=1, seed=1):
    """W[rows,K] fp16 ~ N(0, 0.02^2), x[m,K] fp16 ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.02)).astype(np.float16)
    x = rng.standard_normal((m, K), dtype=np.float32).astype(np.float16)
    return w, x


def c3_gemm(M, N, K, seed=2, batch=None):
    """A[M,K] row-major and B stored [N,K] (column-major KxN), entries N(0,1)/sqrt(K)."""
    rng = np.random.default_rng(seed)
    s = np.float32(1.0 / np.sqrt(K))
    sa = (M, K) if batch is None else (batch, M, K)
    sb = (N, K) if batch is None else (batch, N, K)
    a = (rng.standard_normal(sa, dtype=np.float32) * s).astype(np.float16)
    b = (rng.standard_normal(sb, dtype=np.float32) * s).astype(np.float16)
    return a, b


def c4_conv(batch, IC, H, W, OC, kH, kW, stride, pad, seed=3):
    """x[N,H,W,C] ~ U[-1,1], w[K,R,S,C] ~ N(0, 2/(C*R*S)), both fp16."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, (batch, H, W, IC)).astype(np.float32).astype(np.float16)
    sigma = np.float32(np.sqrt(2.0 / (IC * kH * kW)))
    w = (rng.standard_normal((OC, kH, kW, IC), dtype=np.float32) * sigma).astype(np.float16)
    return x, w


def c5_conv(batch, IC, H, W, OC, kH, kW, stride, pad, seed=4):
    """Model-level sweep data: everything N(0,1)/sqrt(K) with K = IC*kH*kW."""
    rng = np.random.default_rng(seed)
    s = np.float32(1.0 / np.sqrt(IC * kH * kW))
    x = (rng.standard_normal((batch, H, W, IC), dtype=np.float32) * s).astype(np.float16)
    w = (rng.standard_normal((OC, kH, kW, IC), dtype=np.float32) * s).astype(np.float16)
    return x, w
