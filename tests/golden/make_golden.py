"""Generate the golden vectors under tests/golden/ from the reference's own host loops.

Needs ``oracle/_ref`` (``make -C oracle ref``, which compiles the unmodified
reference files src_template/Ampere_FP32/sgemm.cu and src_template/Ampere_FP16/
gemm.cu).  Outputs come from cpuSgemm (sgemm.cu:12-24) and cpuF16F16Gemm
(gemm.cu:26-37); inputs are seeded numpy draws plus the known-answer patterns
the reference harnesses use (uniform [0,1) inputs, gemm.cu:589-593; the
``i/10000`` ramp, gemv.cu:278).  The convolution vectors compose the reference's
conv -> GEMM mapping (scripts/Ampere_FP16/Ampere_FP16_conv.py:432-434), its
im2col layout (src_template/Ampere_FP16/im2col.cu:37-75) and cpuF16F16Gemm.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def sgemm_cases():
    out = {}
    rng = np.random.default_rng(1234)
    for i, (M, N, K) in enumerate([(17, 33, 65), (64, 64, 64), (1, 128, 7), (40, 5, 300)]):
        a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
        out[f"s{i}_a"], out[f"s{i}_b"], out[f"s{i}_c"] = a, b, ref.cpuSgemm(a, b)
    # known answers: identity and all-ones K-sum
    a = rng.uniform(0, 1, (24, 24)).astype(np.float32)
    out["s_id_a"], out["s_id_b"], out["s_id_c"] = a, np.eye(24, dtype=np.float32), ref.cpuSgemm(a, np.eye(24, dtype=np.float32))
    ones_a, ones_b = np.ones((8, 1000), np.float32), np.ones((1000, 8), np.float32)
    out["s_one_a"], out["s_one_b"], out["s_one_c"] = ones_a, ones_b, ref.cpuSgemm(ones_a, ones_b)
    return out


def hgemm_cases():
    out = {}
    rng = np.random.default_rng(4321)
    for i, (M, N, K) in enumerate([(16, 24, 40), (33, 17, 129), (128, 8, 64), (5, 130, 264)]):
        a = rng.uniform(0, 1, (M, K)).astype(np.float32).astype(np.float16)
        b = rng.uniform(0, 1, (K, N)).astype(np.float32).astype(np.float16)
        out[f"h{i}_a"], out[f"h{i}_b_kn"], out[f"h{i}_c"] = a, b, ref.cpuF16F16Gemm(a, b)
    # ramp operand as in the reference's GEMV self-check
    K, N = 256, 16
    a = rng.standard_normal((4, K)).astype(np.float32).astype(np.float16)
    b = (np.arange(K * N, dtype=np.float32) / 10000.0).reshape(K, N).astype(np.float16)
    out["h_ramp_a"], out["h_ramp_b_kn"], out["h_ramp_c"] = a, b, ref.cpuF16F16Gemm(a, b)
    # one-hot rows pick single columns exactly
    a = np.zeros((8, 64), np.float16)
    a[np.arange(8), np.arange(8) * 7] = 1
    b = rng.standard_normal((64, 32)).astype(np.float32).astype(np.float16)
    out["h_hot_a"], out["h_hot_b_kn"], out["h_hot_c"] = a, b, ref.cpuF16F16Gemm(a, b)
    return out


def im2col_nchw(x, k, stride, pad):
    """col[b][c*k*k + i*k + j][ho][wo] with zero padding (im2col.cu:49-69)."""
    B, C, H, W = x.shape
    Ho, Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    xp = np.zeros((B, C, H + 2 * pad, W + 2 * pad), x.dtype)
    xp[:, :, pad:pad + H, pad:pad + W] = x
    col = np.zeros((B, C * k * k, Ho, Wo), x.dtype)
    for c in range(C):
        for i in range(k):
            for j in range(k):
                col[:, c * k * k + i * k + j] = xp[:, c, i:i + Ho * stride:stride, j:j + Wo * stride:stride]
    return col


def conv_cases():
    out = {}
    rng = np.random.default_rng(777)
    for i, (B, C, H, W, OC, k, stride, pad) in enumerate([(2, 8, 9, 9, 16, 3, 1, 1), (1, 16, 12, 10, 8, 3, 2, 1),
                                                          (2, 8, 6, 6, 8, 1, 1, 0), (1, 8, 11, 11, 8, 5, 2, 2),
                                                          # an RGB network's first layer: 3 channels, 7 x 7 / 2, pad 3
                                                          (2, 3, 20, 24, 64, 7, 2, 3),
                                                          # 3 x 3 at 64 -> 64 channels, rows of 50 pixels
                                                          (1, 64, 6, 50, 64, 3, 1, 1)]):
        x = rng.uniform(-1, 1, (B, C, H, W)).astype(np.float32).astype(np.float16)        # NCHW as the reference
        w = (rng.standard_normal((OC, C, k, k)) * np.sqrt(2.0 / (C * k * k))).astype(np.float32).astype(np.float16)
        col = im2col_nchw(x, k, stride, pad)                                              # [B, K, Ho, Wo]
        Ho, Wo = col.shape[2], col.shape[3]
        a = np.ascontiguousarray(col.transpose(0, 2, 3, 1).reshape(B * Ho * Wo, C * k * k))  # M x K
        b_kn = np.ascontiguousarray(w.reshape(OC, C * k * k).T)                              # K x N
        y = ref.cpuF16F16Gemm(a, b_kn).reshape(B, Ho, Wo, OC)                                # NHWC order of M
        out[f"c{i}_x_nchw"], out[f"c{i}_w_oihw"], out[f"c{i}_y_nhwc"] = x, w, y
        out[f"c{i}_geom"] = np.array([B, C, H, W, OC, k, k, stride, pad], np.int32)
    return out


def main():
    if not ref.build():
        raise SystemExit("oracle/_ref is not built and the reference tree is not present")
    np.savez_compressed(os.path.join(HERE, "sgemm_ref.npz"), **sgemm_cases())
    np.savez_compressed(os.path.join(HERE, "hgemm_ref.npz"), **hgemm_cases())
    np.savez_compressed(os.path.join(HERE, "conv_ref.npz"), **conv_cases())
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
