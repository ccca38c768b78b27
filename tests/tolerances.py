"""Acceptance tolerances of the parity tests.

fp32: 1e-5 relative.  fp16: 2e-3 relative or one fp16 ulp (2^-11 relative, 2^-24 absolute in the
subnormal range), whichever is larger.  bf16 has no reference chain and is held to one bf16 ulp
(2^-8 relative) of the fp64 result.  "Relative" is taken against max(|ref|, floor) where the floor
is a tenth of the tensor's RMS, so that elements which are themselves the result of a
cancellation are not held to a tighter bound than the arithmetic that produced them.
Callers that widen the floor (floor_frac = 1.0: relative to the tensor's RMS, for sums of O(1) 16-bit terms that
cancel) or pass a floor of their own are recorded in OVERRIDES together with the number of elements that would have
failed the plain bound; the test session prints that table at its end (tests/conftest.py), so the effect of every
override is on record next to the results.
"""
import numpy as np

RTOL = {"float32": 1e-5, "float16": 2e-3, "bfloat16": 2.0 ** -7}
FLOOR_FRAC = {"float32": 1e-1, "float16": 1e-1, "bfloat16": 1e-1}
ABS_MIN = {"float32": 1e-30, "float16": 2.0 ** -24, "bfloat16": 1e-30}


OVERRIDES = []      # (what, kind, elements, elements outside the plain bound, worst error / plain bound)


def assert_close(got, ref, kind, what="", rtol=None, floor_frac=None, floor_abs=0.0):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    nan_g, nan_r = np.isnan(got), np.isnan(ref)
    assert (nan_g == nan_r).all(), f"{what}: NaN pattern differs"
    got = np.where(nan_r, 0.0, got)
    ref = np.where(nan_r, 0.0, ref)
    rtol = RTOL[kind] if rtol is None else rtol
    ff = FLOOR_FRAC[kind] if floor_frac is None else floor_frac
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    bound = rtol * np.maximum(np.maximum(np.abs(ref), ff * rms), floor_abs) + ABS_MIN[kind]
    err = np.abs(got - ref)
    if ff != FLOOR_FRAC[kind] or np.any(np.asarray(floor_abs) != 0.0) or rtol != RTOL[kind]:
        plain = RTOL[kind] * np.maximum(np.abs(ref), FLOOR_FRAC[kind] * rms) + ABS_MIN[kind]
        OVERRIDES.append((what, kind, int(err.size), int((err > plain).sum()), float((err / plain).max()) if err.size else 0.0))
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err / bound), err.shape)
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.size} out of tolerance; worst at {i}: got {got[i]!r} "
                             f"ref {ref[i]!r} err {err[i]:.3e} bound {bound[i]:.3e}")
