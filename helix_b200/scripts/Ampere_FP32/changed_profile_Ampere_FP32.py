"""Fast profiling mode of the fp32 backend (reference: scripts/Ampere_FP32/changed_profile_Ampere_FP32.py:16-48):
smaller probe problems."""
import _bootstrap  # noqa: F401
from Ampere_FP32.profile_Ampere_FP32 import profile_Helix_Ampere_FP32_gemm_kernel as _full


def profile_Helix_Ampere_FP32_gemm_kernel():
    return _full(fast=True)


if __name__ == "__main__":

    profile_Helix_Ampere_FP32_gemm_kernel()
