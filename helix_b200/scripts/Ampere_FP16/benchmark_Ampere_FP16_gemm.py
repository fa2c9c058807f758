"""Op-level GEMM sweep (reference: scripts/Ampere_FP16/benchmark_Ampere_FP16_gemm.py:9-23)."""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_gemm_op_MNKList
from Ampere_FP16.Ampere_FP16_gemm import get_Ampere_FP16_gemm_cublas_result

root_path = os.getcwd()


def Ampere_FP16_Helix_op_level_GEMM_benchmark(backend="cuda", gpus=1, limit=0, journal=None):
    from helix_b200 import costmodel, harness
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')

    MNKList = get_gemm_op_MNKList()
    if limit:
        MNKList = MNKList[:limit]
    predicted = [harness.predicted_time(prof_dict, harness.cost_model(prof_dict, M, N, K), M, N, K) for M, N, K in MNKList]
    rows = harness.run_shape_list(MNKList, harness.worker_gemm_f16, prof_dict, gpus, predicted, journal=journal)
    for (M, N, K), row in zip(MNKList, rows):
        helix_tflops = row["tflops"]
        print(f'{M}x{N}x{K}: Helix: {helix_tflops:.2f} TFLOPS')
    return rows


def Ampere_FP16_cublas_op_level_GEMM_benchmark(limit=0):
    MNKList = get_gemm_op_MNKList()[:limit or None]
    for M, N, K in MNKList:
        _, cublas_tflops = get_Ampere_FP16_gemm_cublas_result(M, N, K)
        print(f'{M}x{N}x{K}: cublas: {cublas_tflops:.2f} TFLOPS')


if __name__ == "__main__":

    Ampere_FP16_Helix_op_level_GEMM_benchmark(backend="cuda")
    Ampere_FP16_cublas_op_level_GEMM_benchmark()
