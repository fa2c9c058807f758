"""Model-level convolution sweep (reference: scripts/Ampere_FP16/benchmark_Ampere_FP16_model_level_CNN.py:9-48)."""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_cnn_opset_shape_List
from Ampere_FP16.Ampere_FP16_conv import get_Ampere_FP16_conv_cudnn_result

root_path = os.getcwd()


def Ampere_FP16_Helix_model_level_CNN_benchmark(backend="cuda", gpus=1, limit=0, journal=None):
    from helix_b200 import costmodel, harness
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')

    costs = []
    for model_idx, shape_list in enumerate(get_cnn_opset_shape_List()):
        if limit:
            shape_list = shape_list[:limit]
        distinct = sorted(set(shape_list))
        rows = harness.run_shape_list(distinct, harness.worker_conv_f16, prof_dict, gpus, None, journal=(f'{journal}.model{model_idx}' if journal else None))   # one journal per model: indices are per list
        ms = {u: r["ms"] for u, r in zip(distinct, rows)}
        costs.append(sum(ms[u] for u in shape_list))
    helix_AlexNet_cost, helix_ResNet_cost, helix_GoogleNet_cost = costs
    print(f'AlexNet: {helix_AlexNet_cost:.2f} ms, ResNet: {helix_ResNet_cost:.2f} ms, GoogleNet: {helix_GoogleNet_cost:.2f} ms')
    return costs


def Ampere_FP16_cudnn_model_level_CNN_benchmark():
    costs = []
    for shape_list in get_cnn_opset_shape_List():
        distinct = sorted(set(shape_list))
        ms = {u: get_Ampere_FP16_conv_cudnn_result(*u)[0] for u in distinct}
        costs.append(sum(ms[u] for u in shape_list))
    cudnn_AlexNet_cost, cudnn_ResNet_cost, cudnn_GoogleNet_cost = costs
    print(f'AlexNet: {cudnn_AlexNet_cost:.2f} ms, ResNet: {cudnn_ResNet_cost:.2f} ms, GoogleNet: {cudnn_GoogleNet_cost:.2f} ms')


if __name__ == "__main__":

    Ampere_FP16_Helix_model_level_CNN_benchmark(backend="cuda")
    Ampere_FP16_cudnn_model_level_CNN_benchmark()
