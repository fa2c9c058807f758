"""Stand-in for one of the reference's kernel executables, for callers that still parse their stdout.

The reference's scripts spawn ``build/bin_fp16/gemm_<cfg> M N K`` (or ``bin_fp32/sgemm_<cfg>``, ``bin_fp16/gemv``)
and read the average seconds as whitespace token [-8] of the single result line
(src_template/Ampere_FP16/gemm.cu:687-689; scripts/Ampere_FP16/Ampere_FP16_gemm.py:438-441).  This module
prints that line, character for character in the reference's format, from an in-process measurement:

  python -m helix_b200.kernel_exe gemm|gemv|sgemm M N K

so ``os.popen(...).read().split()[-8]`` keeps working against the B200 kernels.  The cuBLAS comparator's
format (token [-4] = milliseconds, [-2] = TFLOP/s; src_template/Ampere_FP16/cublas_f16.cu:101) is printed by
``cublas M N K``.
"""
import sys


def result_line(M, N, K, min_s, avg_s, max_s):
    """The reference executable's result line (gemm.cu:687-689)."""
    tflops = float(M) * N * K * 2 / 1e12 / avg_s
    return "M N K = %6d %6d %6d, Time = %12.8f %12.8f %12.8f s, AVG Performance = %10.4f Tflops" % (
        M, N, K, min_s, avg_s, max_s, tflops)


def cublas_line(M, N, K, ms, tflops):
    """The cuBLAS comparator's line (cublas_f16.cu:101)."""
    return "CBLAS - M : %d, N : %d, K : %d, %f ms, %f Tflops" % (M, N, K, ms, tflops)


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 4 or argv[0] not in ("gemm", "gemv", "sgemm", "cublas"):
        print("usage: python -m helix_b200.kernel_exe gemm|gemv|sgemm|cublas M N K", file=sys.stderr)
        return 2
    kind, (M, N, K) = argv[0], (int(v) for v in argv[1:])
    from . import harness
    harness.require_gpu()
    if kind == "cublas":
        ms, tflops = harness.cublas_gemm_result(M, N, K)
        print(cublas_line(M, N, K, ms, tflops))
        return 0
    if kind == "sgemm":
        times = [harness.time_gemm_f32(M, N, K) for _ in range(3)]
    elif kind == "gemv":
        Kp = (K + 7) // 8 * 8
        rows, m, transposed = (N, M, False) if M <= N else (M, N, True)
        times = [harness.time_gemv_f16(rows, Kp, m, None, transposed) for _ in range(3)]
    else:
        times = [harness.time_gemm_f16(M, N, (K + 7) // 8 * 8) for _ in range(3)]
    print(result_line(M, N, K, min(times), sum(times) / len(times), max(times)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
