"""Selection + execution of one fp16 convolution (reference: scripts/Ampere_FP16/Ampere_FP16_conv.py:419-559)."""
import os

import _bootstrap  # noqa: F401

root_path = os.getcwd()


def cost_model(prof_dict, M, N, K):
    from helix_b200 import costmodel
    return costmodel.cost_model(prof_dict, M, N, K, conv=True)


def get_Ampere_FP16_conv_Helix_result(prof_dict, batch, input_channel, H, W, output_channel, kH, kW, stride, pad, backend="cuda"):
    if backend != "cuda":
        raise ValueError("only backend='cuda' is available (no TVM code generation in this build)")
    from helix_b200 import harness
    return harness.conv_f16_result(prof_dict, batch, input_channel, H, W, output_channel, kH, kW, stride, pad)


def get_Ampere_FP16_conv_cudnn_result(batch, input_channel, H, W, output_channel, kH, kW, stride, pad):
    from helix_b200 import harness
    return harness.cudnn_conv_result(batch, input_channel, H, W, output_channel, kH, kW, stride, pad)
