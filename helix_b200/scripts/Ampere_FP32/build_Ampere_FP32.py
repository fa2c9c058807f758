"""Generator step of the fp32 backend (reference: scripts/Ampere_FP32/build_Ampere_FP32.py:37-80).

The reference launches 2 538 un-awaited nvcc processes, one per (BM, BN, BK, TM, TN, ...) tuple; here the
SIMT FFMA tiles are template instantiations of one library and build/bin_fp32/ keeps a manifest."""
import os

import _bootstrap  # noqa: F401
from tqdm import tqdm

root_path = os.getcwd()


def is_valid_config(BMt, BNt, BM, BN):
    """Same predicate as the reference's (build_Ampere_FP32.py:7-12), applied to the tiles compiled in."""
    if BMt * BNt * 32 >= 512:
        return False
    if BM > 128 or BN > 128 or BM < 4 or BN < 4:
        return False
    return True


def get_copy_value(base_value, threshold=4):
    return base_value if base_value < threshold else threshold


def compile_sgemm(*_):
    from helix_b200 import build
    return build.build()


def build_Helix_Ampere_FP32_gemm_kernel():
    from helix_b200 import costmodel
    os.makedirs(f"{root_path}/build/bin_fp32", exist_ok=True)
    print("Start building Ampere FP32 GEMM kernel ...")
    keys = costmodel.sgemm_keys()
    with tqdm(total=len(keys) + 1, desc="building") as pbar:
        lib = compile_sgemm()
        pbar.update(1)
        with open(f"{root_path}/build/bin_fp32/MANIFEST", "w") as f:
            f.write(f"# configurations inside {lib}\n")
            for k in keys:
                f.write("sgemm_" + "_".join(str(v) for v in k) + "\n")
                pbar.update(1)
    print("Build finished.")


def build_cublas_FP32_gemm_kernel():
    os.makedirs(f"{root_path}/build/bin_fp32", exist_ok=True)


def build_cudnn_FP32_conv_kernel():
    """Named as scripts/build_template.py:4 imports it (the reference defines it under another name)."""
    os.makedirs(f"{root_path}/build/bin_fp32", exist_ok=True)


if __name__ == "__main__":

    build_Helix_Ampere_FP32_gemm_kernel()
    build_cublas_FP32_gemm_kernel()
    build_cudnn_FP32_conv_kernel()
