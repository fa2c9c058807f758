"""Selection + execution of one fp32 GEMM (reference: scripts/Ampere_FP32/Ampere_FP32_gemm.py:89-146)."""
import os

import _bootstrap  # noqa: F401

root_path = os.getcwd()


def cost_model(prof_dict, M, N, K):
    from helix_b200 import costmodel
    return costmodel.sgemm_cost_model(prof_dict, M, N, K)


def get_Ampere_FP32_gemm_Helix_result(prof_dict, M, N, K, backend="cuda"):
    if backend != "cuda":
        raise ValueError("only backend='cuda' is available (no TVM code generation in this build)")
    from helix_b200 import harness
    return harness.gemm_f32_result(prof_dict, M, N, K)


def get_Ampere_FP32_gemm_cublas_result(M, N, K):
    import torch
    from helix_b200 import harness
    return harness.cublas_gemm_result(M, N, K, dtype=torch.float32)
