"""Selection overhead vs. op time (reference: scripts/Ampere_FP16/Ampere_FP16_runtime_cost.py:7-40)."""
import os
import time

import _bootstrap  # noqa: F401

root_path = os.getcwd()


def cost_model(prof_dict, M, N, K):
    from helix_b200 import harness
    return harness.cost_model(prof_dict, M, N, K)


def get_Helix_runtime_cost(prof_dict, M, N, K):
    from helix_b200 import harness
    T1 = time.perf_counter()
    for i in range(100):
        best_config = cost_model(prof_dict, M, N, K)
    T2 = time.perf_counter()
    if best_config[0] == 0:
        rows, m, tr = (N, M, False) if M <= N else (M, N, True)
        cost = harness.time_gemv_f16(rows, K, m, harness.key_to_cfg(best_config), tr)
    else:
        cost = harness.time_gemm_f16(M, N, K, harness.key_to_cfg(best_config))
    # same units as the reference's print: selection overhead per call (its /100/1000 scaling) and op seconds
    return (T2 - T1) / 100 / 1000, cost


def Ampere_FP16_runtime_cost():
    from helix_b200 import costmodel
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')

    MNKList = [(64, 64, 64), (128, 128, 128), (256, 256, 256), (512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096)]
    for M, N, K in MNKList:
        runtime_cost, op_cost = get_Helix_runtime_cost(prof_dict, M, N, K)
        print(f'The runtime cost of {M}x{N}x{K} is {runtime_cost} ms, and the op cost is {op_cost} ms.')


if __name__ == '__main__':

    Ampere_FP16_runtime_cost()
