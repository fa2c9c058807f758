"""CLI of the fast profiling mode (reference: scripts/changed_profile.py:9-24)."""
import argparse
import time

import _bootstrap  # noqa: F401

if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Get runtime cost of an operation")
    parser.add_argument("-b", "--backend", type=str, choices=['Ampere_FP16', 'Ampere_FP32', 'x86_CPU', 'ARM_CPU'], default='Ampere_FP16', help="backend")
    args = parser.parse_args()

    T1 = time.perf_counter()
    if args.backend == 'Ampere_FP16':
        from Ampere_FP16.changed_profile_Ampere_FP16 import profile_Helix_Ampere_FP16_gemm_kernel
        profile_Helix_Ampere_FP16_gemm_kernel()
    elif args.backend == 'Ampere_FP32':
        from Ampere_FP32.changed_profile_Ampere_FP32 import profile_Helix_Ampere_FP32_gemm_kernel
        profile_Helix_Ampere_FP32_gemm_kernel()
    else:
        print(f"{args.backend} is the reference's TVM-generated CPU backend; this build covers the GPU backends only")
    T2 = time.perf_counter()
    print(f'Profiling time: {T2-T1} seconds')
