"""Selection ablation over the op-level GEMM list: exhaustive best ("Oracle") against the cost model's
pick ("Default") and two static policies
(reference: scripts/Ampere_FP16/benchmark_Ampere_FP16_performance_comparison.py:8-113).

The reference's static policies restrict the candidate set (Static1: tiles whose warp tile equals the CTA
tile) or ignore the shape (Static2: the candidate with the smallest profiled time).  Their counterparts
here: Static1 keeps only the plain one-CTA kernel (no operand swap, no K split, no CTA pair) and
Static2 always runs the configuration with the smallest profiled time per K slab.
"""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_gemm_op_MNKList

root_path = os.getcwd()


def _kernel_keys(prof_dict):
    return [k for k in prof_dict if len(k) == 6]


def cost_model(prof_dict, M, N, K):
    from helix_b200 import harness
    return harness.cost_model(prof_dict, M, N, K)


def cost_model_static1(prof_dict, M, N, K):
    from helix_b200 import harness
    plain = {k: v for k, v in prof_dict.items()
             if len(k) != 6 or (k[0] != 0 and k[3] == 1 and k[4] == 0 and k[5] == 0)}
    return harness.cost_model(plain, M, N, K)


def cost_model_static2(prof_dict, M, N, K):
    """Shape-blind: the tensor-core key with the smallest profiled seconds per K slab that can run at all."""
    from helix_b200 import harness
    best, best_key = float("inf"), None
    for k in _kernel_keys(prof_dict):
        if k[0] == 0 or harness.predicted_time(prof_dict, k, M, N, K) == float("inf"):
            continue
        per_slab = prof_dict[k][1] / (k[1] * k[2] * k[3])       # seconds per slab per output element
        if per_slab < best:
            best, best_key = per_slab, k
    return best_key


def _tflops(key, M, N, K):
    from helix_b200 import harness
    return 2 * M * N * K / 1e12 / harness.time_key_f16(key, M, N, K)


def get_Helix_Default_result(prof_dict, M, N, K):
    return _tflops(cost_model(prof_dict, M, N, K), M, N, K)


def get_Helix_Oracle_result(prof_dict, M, N, K):
    from helix_b200 import harness
    best = 0.0
    for k in _kernel_keys(prof_dict):
        if k[0] == 0 and min(M, N) > 8:
            continue
        if harness.predicted_time(prof_dict, k, M, N, K) == float("inf"):
            continue
        best = max(best, _tflops(k, M, N, K))
    return best


def get_Helix_Static1_result(prof_dict, M, N, K):
    return _tflops(cost_model_static1(prof_dict, M, N, K), M, N, K)


def get_Helix_Static2_result(prof_dict, M, N, K):
    return _tflops(cost_model_static2(prof_dict, M, N, K), M, N, K)


def performance_comparison(prof_dict, MNKList, out=print):
    rows = []
    for M, N, K in MNKList:
        helix_oracle_flops = get_Helix_Oracle_result(prof_dict, M, N, K)
        helix_default_flops = get_Helix_Default_result(prof_dict, M, N, K)
        helix_static1_flops = get_Helix_Static1_result(prof_dict, M, N, K)
        helix_static2_flops = get_Helix_Static2_result(prof_dict, M, N, K)
        rows.append((M, N, K, helix_oracle_flops, helix_default_flops, helix_static1_flops, helix_static2_flops))
        out(f'{M}x{N}x{K}: Helix_Oracle: {helix_oracle_flops:.2f} TFlops, Helix_Default: {helix_default_flops:.2f} TFlops, '
            f'Helix_Static1: {helix_static1_flops:.2f} TFlops, Helix_Static2: {helix_static2_flops:.2f} TFlops')
    return rows


if __name__ == "__main__":
    import argparse
    from helix_b200 import costmodel
    ap = argparse.ArgumentParser()
    ap.add_argument("--limit", type=int, default=0, help="only the first N shapes of the op-level list (0 = all)")
    ap.add_argument("--stride", type=int, default=1, help="take every n-th shape of the list")
    args = ap.parse_args()
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')
    MNKList = get_gemm_op_MNKList()[::max(1, args.stride)]
    if args.limit:
        MNKList = MNKList[:args.limit]
    performance_comparison(prof_dict, MNKList)
