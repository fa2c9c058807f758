"""Error metrics shared by the parity tests.

Tolerances: fp16 results need relative Frobenius error <= 2e-3 and max
element-wise relative error <= 1e-2 over outputs with |y| > 1e-3; fp32 results
need relative error <= 1e-5.
"""
import numpy as np

F16_FRO_TOL = 2e-3
F16_ELEM_TOL = 1e-2
F32_TOL = 1e-5
ELEM_FLOOR = 1e-3


def rel_fro(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((got - ref).ravel()) / (den if den > 0 else 1.0))


def max_elem_rel(got, ref, floor=ELEM_FLOOR):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    mask = np.abs(ref) > floor
    if not mask.any():
        return 0.0
    return float(np.max(np.abs(got[mask] - ref[mask]) / np.abs(ref[mask])))


def assert_f16_close(got, ref32, what=""):
    """``got``: fp16 result; ``ref32``: the oracle's unrounded fp32 sums."""
    assert np.isfinite(np.asarray(got, dtype=np.float32)).all(), f"{what}: non-finite output"
    fro = rel_fro(got, ref32)
    mx = max_elem_rel(got, ref32)
    assert fro <= F16_FRO_TOL, f"{what}: relative Frobenius error {fro:.3e} > {F16_FRO_TOL}"
    assert mx <= F16_ELEM_TOL, f"{what}: max element-wise relative error {mx:.3e} > {F16_ELEM_TOL}"
    return fro, mx


def assert_f32_close(got, ref, what=""):
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    fro = rel_fro(got, ref)
    assert fro <= F32_TOL, f"{what}: relative Frobenius error {fro:.3e} > {F32_TOL}"
    return fro
