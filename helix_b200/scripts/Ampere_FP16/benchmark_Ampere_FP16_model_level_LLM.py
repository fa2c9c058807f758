"""Model-level GEMM sweep (reference: scripts/Ampere_FP16/benchmark_Ampere_FP16_model_level_LLM.py:9-48)."""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_llm_opset_MNKList
from Ampere_FP16.Ampere_FP16_gemm import get_Ampere_FP16_gemm_cublas_result

root_path = os.getcwd()


def Ampere_FP16_Helix_model_level_LLM_benchmark(backend="cuda", gpus=1, limit=0, journal=None):
    from helix_b200 import costmodel, harness
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')

    lists = get_llm_opset_MNKList()
    costs = []
    for model_idx, MNKList in enumerate(lists):
        if limit:
            MNKList = MNKList[:limit]
        # identical shapes repeat many times inside a model: measure each distinct shape once
        distinct = sorted(set(MNKList))
        rows = harness.run_shape_list(distinct, harness.worker_gemm_f16, prof_dict, gpus, None, journal=(f'{journal}.model{model_idx}' if journal else None))   # one journal per model: indices are per list
        ms = {u: r["ms"] for u, r in zip(distinct, rows)}
        costs.append(sum(ms[u] for u in MNKList))
    helix_Bert_cost, helix_LLAMA2_cost, helix_GPT2_cost = costs
    print(f'Bert: {helix_Bert_cost:.2f} ms, LLAMA2: {helix_LLAMA2_cost:.2f} ms, GPT2: {helix_GPT2_cost:.2f} ms')
    return costs


def Ampere_FP16_cublas_model_level_LLM_benchmark():
    costs = []
    for MNKList in get_llm_opset_MNKList():
        distinct = sorted(set(MNKList))
        ms = {u: get_Ampere_FP16_gemm_cublas_result(*u)[0] for u in distinct}
        costs.append(sum(ms[u] for u in MNKList))
    cublas_Bert_cost, cublas_LLAMA2_cost, cublas_GPT2_cost = costs
    print(f'Bert: {cublas_Bert_cost:.2f} ms, LLAMA2: {cublas_LLAMA2_cost:.2f} ms, GPT2: {cublas_GPT2_cost:.2f} ms')


if __name__ == "__main__":

    Ampere_FP16_Helix_model_level_LLM_benchmark(backend="cuda")
    Ampere_FP16_cublas_model_level_LLM_benchmark()
