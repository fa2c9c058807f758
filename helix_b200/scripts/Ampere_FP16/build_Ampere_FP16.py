"""Generator step of the fp16 backend (reference: scripts/Ampere_FP16/build_Ampere_FP16.py:41-86).

The reference compiles one executable per (K_STAGE, BLOCK, WARP) tuple (787 nvcc runs).  Here every
configuration is a template instantiation inside libhelix_b200.so, built once (in parallel, cached by
content hash); build/bin_fp16/ keeps a manifest naming the configurations in the reference's style."""
import os

import _bootstrap  # noqa: F401
from tqdm import tqdm

root_path = os.getcwd()


def is_valid_config(tile_n, swap_ab, mode, stages=0):
    from helix_b200 import costmodel
    return costmodel.is_valid_config(tile_n, swap_ab, mode, stages)


def compile_kernel(kernel_name=None, *_):
    """All kernels live in one library; compiling any of them builds it (no per-configuration nvcc run)."""
    from helix_b200 import build
    return build.build()


def build_Helix_Ampere_FP16_gemm_kernel():
    from helix_b200 import costmodel
    os.makedirs(f"{root_path}/build/bin_fp16", exist_ok=True)
    print("Start building Ampere FP16 GEMM kernel ...")
    keys = costmodel.gemm_keys() + costmodel.gemv_keys()
    with tqdm(total=len(keys) + 1, desc="building") as pbar:
        lib = compile_kernel()
        pbar.update(1)
        with open(f"{root_path}/build/bin_fp16/MANIFEST", "w") as f:
            f.write(f"# configurations inside {lib}\n")
            for k in keys:
                name = ("gemv" if k[0] == 0 else "gemm") + "_" + "_".join(str(v) for v in k)
                f.write(name + "\n")
                pbar.update(1)
    print("Build finished.")


def build_cublas_FP16_gemm_kernel():
    """The cuBLAS comparator needs no build: it is timed through torch.matmul."""
    os.makedirs(f"{root_path}/build/bin_fp16", exist_ok=True)


def build_cudnn_FP16_conv_kernel():
    """The cuDNN comparator needs no build: it is timed through torch's conv2d."""
    os.makedirs(f"{root_path}/build/bin_fp16", exist_ok=True)


if __name__ == "__main__":

    build_Helix_Ampere_FP16_gemm_kernel()
    build_cublas_FP16_gemm_kernel()
    build_cudnn_FP16_conv_kernel()
