"""CLI of the generator step (reference: scripts/build_template.py:6-18).  Backend imports are lazy,
so one backend's missing dependency cannot break the other (the reference imports all eagerly)."""
import argparse

import _bootstrap  # noqa: F401

if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Get runtime cost of an operation")
    parser.add_argument("-b", "--backend", type=str, choices=['Ampere_FP16', 'Ampere_FP32'], default='Ampere_FP16', help="backend")
    args = parser.parse_args()

    if args.backend == 'Ampere_FP16':
        from Ampere_FP16.build_Ampere_FP16 import (build_Helix_Ampere_FP16_gemm_kernel, build_cublas_FP16_gemm_kernel,
                                                    build_cudnn_FP16_conv_kernel)
        build_Helix_Ampere_FP16_gemm_kernel()
        build_cublas_FP16_gemm_kernel()
        build_cudnn_FP16_conv_kernel()
    elif args.backend == 'Ampere_FP32':
        from Ampere_FP32.build_Ampere_FP32 import (build_Helix_Ampere_FP32_gemm_kernel, build_cublas_FP32_gemm_kernel,
                                                    build_cudnn_FP32_conv_kernel)
        build_Helix_Ampere_FP32_gemm_kernel()
        build_cublas_FP32_gemm_kernel()
        build_cudnn_FP32_conv_kernel()
