"""Model-level fp32 GEMM sweep (reference: scripts/Ampere_FP32/benchmark_Ampere_FP32_model_level_LLM.py:9-48)."""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_llm_opset_MNKList
from Ampere_FP32.Ampere_FP32_gemm import get_Ampere_FP32_gemm_cublas_result

root_path = os.getcwd()


def Ampere_FP32_Helix_model_level_LLM_benchmark(backend="cuda", gpus=1, limit=0, journal=None):
    from helix_b200 import costmodel, harness
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP32_cost_model.dict')
    costs = []
    for model_idx, MNKList in enumerate(get_llm_opset_MNKList()):
        if limit:
            MNKList = MNKList[:limit]
        distinct = sorted(set(MNKList))
        rows = harness.run_shape_list(distinct, harness.worker_gemm_f32, prof_dict, gpus, None, journal=(f'{journal}.model{model_idx}' if journal else None))   # one journal per model: indices are per list
        ms = {u: r["ms"] for u, r in zip(distinct, rows)}
        costs.append(sum(ms[u] for u in MNKList))
    helix_Bert_cost, helix_LLAMA2_cost, helix_GPT2_cost = costs
    print(f'Bert: {helix_Bert_cost:.2f} ms, LLAMA2: {helix_LLAMA2_cost:.2f} ms, GPT2: {helix_GPT2_cost:.2f} ms')
    return costs


def Ampere_FP32_cublas_model_level_LLM_benchmark():
    costs = []
    for MNKList in get_llm_opset_MNKList():
        distinct = sorted(set(MNKList))
        ms = {u: get_Ampere_FP32_gemm_cublas_result(*u)[0] for u in distinct}
        costs.append(sum(ms[u] for u in MNKList))
    cublas_Bert_cost, cublas_LLAMA2_cost, cublas_GPT2_cost = costs
    print(f'Bert: {cublas_Bert_cost:.2f} ms, LLAMA2: {cublas_LLAMA2_cost:.2f} ms, GPT2: {cublas_GPT2_cost:.2f} ms')


if __name__ == "__main__":

    Ampere_FP32_Helix_model_level_LLM_benchmark(backend="cuda")
    Ampere_FP32_cublas_model_level_LLM_benchmark()
