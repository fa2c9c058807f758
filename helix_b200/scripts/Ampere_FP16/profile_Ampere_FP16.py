"""Profiling step of the fp16 backend (reference: scripts/Ampere_FP16/profile_Ampere_FP16.py:17-62):
fills build/prof_dict/Ampere_FP16_cost_model.dict, in-process, through the C ABI."""
import os

import _bootstrap  # noqa: F401
from tqdm import tqdm

root_path = os.getcwd()


def profile_Helix_Ampere_FP16_gemm_kernel(fast=False):
    from helix_b200 import costmodel, harness
    os.makedirs(f"{root_path}/build/prof_dict", exist_ok=True)
    print("Start profiling Ampere FP16 GEMM kernel ...")
    with tqdm(desc="profiling") as pbar:
        prof_dict = harness.profile_fp16(fast=fast, progress=lambda: pbar.update(1))
    costmodel.save(prof_dict, f'{root_path}/build/prof_dict/Ampere_FP16_cost_model.dict')
    print("Profile finished.")
    return prof_dict


if __name__ == "__main__":

    profile_Helix_Ampere_FP16_gemm_kernel()
