"""Fast profiling mode (reference: scripts/Ampere_FP16/changed_profile_Ampere_FP16.py:17-71): probe a
subset of the tile widths and fill the rest by interpolation."""
import _bootstrap  # noqa: F401
from Ampere_FP16.profile_Ampere_FP16 import profile_Helix_Ampere_FP16_gemm_kernel as _full


def profile_Helix_Ampere_FP16_gemm_kernel():
    return _full(fast=True)


if __name__ == "__main__":

    profile_Helix_Ampere_FP16_gemm_kernel()
