"""Op-level sweep CLI (reference: scripts/benchmark_op_level_eval.py:12-45).  `--gpus N` shards the
shape list over N GPUs of the box (one worker process per GPU, LPT on predicted cost)."""
import argparse

import _bootstrap  # noqa: F401


def _table():
    from Ampere_FP16.benchmark_Ampere_FP16_gemm import Ampere_FP16_Helix_op_level_GEMM_benchmark, Ampere_FP16_cublas_op_level_GEMM_benchmark
    from Ampere_FP16.benchmark_Ampere_FP16_conv import Ampere_FP16_Helix_op_level_Conv_benchmark, Ampere_FP16_cudnn_op_level_Conv_benchmark
    from Ampere_FP32.benchmark_Ampere_FP32_gemm import Ampere_FP32_Helix_op_level_GEMM_benchmark, Ampere_FP32_cublas_op_level_GEMM_benchmark
    from Ampere_FP32.benchmark_Ampere_FP32_conv import Ampere_FP32_Helix_op_level_Conv_benchmark, Ampere_FP32_cudnn_op_level_Conv_benchmark
    return {
        ('GEMM', 'Ampere_FP16', 'Helix'): Ampere_FP16_Helix_op_level_GEMM_benchmark,
        ('GEMM', 'Ampere_FP16', 'cublas'): Ampere_FP16_cublas_op_level_GEMM_benchmark,
        ('Conv', 'Ampere_FP16', 'Helix'): Ampere_FP16_Helix_op_level_Conv_benchmark,
        ('Conv', 'Ampere_FP16', 'cudnn'): Ampere_FP16_cudnn_op_level_Conv_benchmark,
        ('GEMM', 'Ampere_FP32', 'Helix'): Ampere_FP32_Helix_op_level_GEMM_benchmark,
        ('GEMM', 'Ampere_FP32', 'cublas'): Ampere_FP32_cublas_op_level_GEMM_benchmark,
        ('Conv', 'Ampere_FP32', 'Helix'): Ampere_FP32_Helix_op_level_Conv_benchmark,
        ('Conv', 'Ampere_FP32', 'cudnn'): Ampere_FP32_cudnn_op_level_Conv_benchmark,
    }


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Benchmark OP level performance")
    parser.add_argument("-o", "--op", type=str, choices=['GEMM', 'Conv'], default='GEMM', help="op type")
    parser.add_argument("-b", "--backend", type=str, choices=['Ampere_FP16', 'Ampere_FP32', 'x86_CPU', 'ARM_CPU'], default='Ampere_FP16', help="backend")
    parser.add_argument("-s", "--system", type=str, choices=['Helix', 'cublas', 'cudnn', 'cutlass', 'DietCode', 'onnxruntime', 'MKL', 'oneDNN', 'ACL'], default='Helix', help="system")
    parser.add_argument("--gpus", type=int, default=1, help="GPUs of this box to shard the shape list over")
    parser.add_argument("--limit", type=int, default=0, help="only the first N shapes (0 = all)")
    parser.add_argument("--journal", type=str, default=None,
                        help="JSONL file: one row per finished shape is appended; shapes found there are not run again")
    args = parser.parse_args()

    func_dict = _table() if args.backend in ('Ampere_FP16', 'Ampere_FP32') else {}
    if (args.op, args.backend, args.system) in func_dict.keys():
        fn = func_dict[(args.op, args.backend, args.system)]
        if args.system == 'Helix':
            fn(gpus=args.gpus, limit=args.limit, journal=args.journal)
        else:
            fn(limit=args.limit)
    else:
        print(f'{args.op} {args.backend} {args.system} is not supported')
