"""Where the memory-bound GEMV kernel hands over to the tensor-core GEMM as M grows
(reference: scripts/Ampere_FP16/TensorCore_CUDACore_Adaptive.py:8-76).

For M in 1..16 and N in {1024, 2048, 4096} at K = 1024 it prints the throughput of the cost model's pick
("Helix"), of the GEMV kernel alone (ceil(M/8) passes of at most 8 right-hand sides) and of the best
tensor-core configuration alone.
"""
import os

import _bootstrap  # noqa: F401

root_path = os.getcwd()


def cost_model(prof_dict, M, N, K):
    from helix_b200 import harness
    return harness.cost_model(prof_dict, M, N, K)


def cost_model_without_gemv(prof_dict, M, N, K):
    """The reference's variant that skips the GEMV keys (TensorCore_CUDACore_Adaptive.py:21-34)."""
    from helix_b200 import harness
    return harness.cost_model({k: v for k, v in prof_dict.items() if not (len(k) == 6 and k[0] == 0)}, M, N, K)


def cost_model_gemv_only(prof_dict, M, N, K):
    from helix_b200 import harness
    gemv = {k: v for k, v in prof_dict.items() if len(k) != 6 or k[0] == 0}
    return harness.cost_model(gemv, min(M, 8), N, K)


def get_Helix_result(prof_dict, M, N, K):
    from helix_b200 import harness
    t = harness.time_key_f16(cost_model(prof_dict, M, N, K), M, N, K)
    return 2 * M * N * K / 1e12 / t


def get_gemv_result(prof_dict, M, N, K):
    from helix_b200 import harness
    key = cost_model_gemv_only(prof_dict, M, N, K)
    t = harness.gemv_passes_time(M, N, K, harness.key_to_cfg(key))
    return 2 * M * N * K / 1e12 / t


def get_gemm_result(prof_dict, M, N, K):
    from helix_b200 import harness
    t = harness.time_key_f16(cost_model_without_gemv(prof_dict, M, N, K), M, N, K)
    return 2 * M * N * K / 1e12 / t


def adaptive_table(prof_dict, MNKList=None, out=print):
    MNKList = MNKList or [(m, n, 1024) for n in [1024, 2048, 4096] for m in [1, 2, 4, 6, 8, 10, 12, 14, 16]]
    rows = []
    for M, N, K in MNKList:
        helix_tflops = get_Helix_result(prof_dict, M, N, K)
        gemv_tflops = get_gemv_result(prof_dict, M, N, K)
        gemm_tflops = get_gemm_result(prof_dict, M, N, K)
        rows.append((M, N, K, helix_tflops, gemv_tflops, gemm_tflops))
        out(f'{M}x{N}x{K}: Helix {helix_tflops:.2f} TFLOPS, Gemv {gemv_tflops:.2f} TFLOPS, GEMM {gemm_tflops:.2f} TFLOPS')
    return rows


if __name__ == "__main__":
    from helix_b200 import costmodel
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')
    adaptive_table(prof_dict)
