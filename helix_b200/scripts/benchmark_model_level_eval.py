"""Model-level sweep CLI (reference: scripts/benchmark_model_level_eval.py:12-45)."""
import argparse

import _bootstrap  # noqa: F401


def _table():
    from Ampere_FP16.benchmark_Ampere_FP16_model_level_LLM import Ampere_FP16_Helix_model_level_LLM_benchmark, Ampere_FP16_cublas_model_level_LLM_benchmark
    from Ampere_FP16.benchmark_Ampere_FP16_model_level_CNN import Ampere_FP16_Helix_model_level_CNN_benchmark, Ampere_FP16_cudnn_model_level_CNN_benchmark
    from Ampere_FP32.benchmark_Ampere_FP32_model_level_LLM import Ampere_FP32_Helix_model_level_LLM_benchmark, Ampere_FP32_cublas_model_level_LLM_benchmark
    from Ampere_FP32.benchmark_Ampere_FP32_model_level_CNN import Ampere_FP32_Helix_model_level_CNN_benchmark, Ampere_FP32_cudnn_model_level_CNN_benchmark
    return {
        ('LLM', 'Ampere_FP16', 'Helix'): Ampere_FP16_Helix_model_level_LLM_benchmark,
        ('LLM', 'Ampere_FP16', 'cublas'): Ampere_FP16_cublas_model_level_LLM_benchmark,
        ('CNN', 'Ampere_FP16', 'Helix'): Ampere_FP16_Helix_model_level_CNN_benchmark,
        # the reference registers the cuDNN runs under 'cublas' (benchmark_model_level_eval.py:16,20); both keys work here
        ('CNN', 'Ampere_FP16', 'cublas'): Ampere_FP16_cudnn_model_level_CNN_benchmark,
        ('CNN', 'Ampere_FP16', 'cudnn'): Ampere_FP16_cudnn_model_level_CNN_benchmark,
        ('LLM', 'Ampere_FP32', 'Helix'): Ampere_FP32_Helix_model_level_LLM_benchmark,
        ('LLM', 'Ampere_FP32', 'cublas'): Ampere_FP32_cublas_model_level_LLM_benchmark,
        ('CNN', 'Ampere_FP32', 'Helix'): Ampere_FP32_Helix_model_level_CNN_benchmark,
        ('CNN', 'Ampere_FP32', 'cublas'): Ampere_FP32_cudnn_model_level_CNN_benchmark,
        ('CNN', 'Ampere_FP32', 'cudnn'): Ampere_FP32_cudnn_model_level_CNN_benchmark,
    }


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description="Benchmark Model level performance")
    parser.add_argument("-m", "--model", type=str, choices=['LLM', 'CNN'], default='LLM', help="model name")
    parser.add_argument("-b", "--backend", type=str, choices=['Ampere_FP16', 'Ampere_FP32', 'x86_CPU', 'ARM_CPU'], default='Ampere_FP16', help="backend")
    parser.add_argument("-s", "--system", type=str, choices=['Helix', 'cublas', 'cudnn', 'cutlass', 'DietCode', 'onnxruntime', 'MKL', 'acl'], default='Helix', help="system")
    parser.add_argument("--gpus", type=int, default=1, help="GPUs of this box to shard the shape lists over")
    parser.add_argument("--limit", type=int, default=0, help="only the first N shapes of each list (0 = all)")
    args = parser.parse_args()

    func_dict = _table() if args.backend in ('Ampere_FP16', 'Ampere_FP32') else {}
    if (args.model, args.backend, args.system) in func_dict.keys():
        fn = func_dict[(args.model, args.backend, args.system)]
        if args.system == 'Helix':
            fn(gpus=args.gpus, limit=args.limit, journal=args.journal)
        else:
            fn()
    else:
        print(f'{args.model} {args.backend} {args.system} is not supported')
