"""Op-level fp32 convolution sweep (reference: scripts/Ampere_FP32/benchmark_Ampere_FP32_conv.py:9-23)."""
import os

import _bootstrap  # noqa: F401
from utils.get_benchmark_shape_list import get_conv_op_shape_list
from Ampere_FP32.Ampere_FP32_conv import get_Ampere_FP32_conv_cudnn_result

root_path = os.getcwd()


def Ampere_FP32_Helix_op_level_Conv_benchmark(backend="cuda", gpus=1, limit=0, journal=None):
    from helix_b200 import costmodel, harness
    prof_dict = costmodel.load(f'{root_path}/build/prof_dict/Ampere_FP32_cost_model.dict')

    shape_list = get_conv_op_shape_list()
    if limit:
        shape_list = shape_list[:limit]
    rows = harness.run_shape_list(shape_list, harness.worker_conv_f32, prof_dict, gpus, None, journal=journal)
    for (batch, input_channel, H, W, output_channel, kH, kW, stride, pad), row in zip(shape_list, rows):
        helix_tflops = row["tflops"]
        print(f'{batch}x{input_channel}x{H}x{W}x{output_channel}x{kH}x{kW}x{stride}x{pad}: Helix: {helix_tflops:.2f} TFLOPS')
    return rows


def Ampere_FP32_cudnn_op_level_Conv_benchmark(limit=0):
    for shape in get_conv_op_shape_list()[:limit or None]:
        _, cudnn_tflops = get_Ampere_FP32_conv_cudnn_result(*shape)
        print('x'.join(str(v) for v in shape) + f': cudnn: {cudnn_tflops:.2f} TFLOPS')


if __name__ == "__main__":

    Ampere_FP32_Helix_op_level_Conv_benchmark(backend="cuda")
    Ampere_FP32_cudnn_op_level_Conv_benchmark()
