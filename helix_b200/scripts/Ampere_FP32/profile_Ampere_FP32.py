"""Profiling step of the fp32 backend (reference: scripts/Ampere_FP32/profile_Ampere_FP32.py:16-51)."""
import os

import _bootstrap  # noqa: F401
from tqdm import tqdm

root_path = os.getcwd()


def profile_Helix_Ampere_FP32_gemm_kernel(fast=False):
    from helix_b200 import costmodel, harness
    os.makedirs(f"{root_path}/build/prof_dict", exist_ok=True)
    print("Start profiling Ampere FP32 GEMM kernel ...")
    with tqdm(total=len(costmodel.sgemm_keys()), desc="profiling") as pbar:
        prof_dict = harness.profile_fp32(fast=fast, progress=lambda: pbar.update(1))
    costmodel.save(prof_dict, f'{root_path}/build/prof_dict/Ampere_FP32_cost_model.dict')
    print("Profile finished.")
    return prof_dict


if __name__ == "__main__":

    profile_Helix_Ampere_FP32_gemm_kernel()
