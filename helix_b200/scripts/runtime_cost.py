"""CLI that reports selection overhead and op time (reference: scripts/runtime_cost.py:8-22)."""
import argparse

import _bootstrap  # noqa: F401

if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Get runtime cost of an operation")
    parser.add_argument("-b", "--backend", type=str, choices=['Ampere_FP16', 'Ampere_FP32', 'x86_CPU', 'ARM_CPU'], default='Ampere_FP16', help="backend")
    args = parser.parse_args()

    if args.backend == 'Ampere_FP16':
        from Ampere_FP16.Ampere_FP16_runtime_cost import Ampere_FP16_runtime_cost
        Ampere_FP16_runtime_cost()
    elif args.backend == 'Ampere_FP32':
        from Ampere_FP32.Ampere_FP32_runtime_cost import Ampere_FP32_runtime_cost
        Ampere_FP32_runtime_cost()
    elif args.backend in ('x86_CPU', 'ARM_CPU'):
        print(f"{args.backend} is the reference's TVM-generated CPU backend; this build covers the GPU backends only")
    else:
        raise ValueError("Invalid backend")
