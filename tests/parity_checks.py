"""Shared checks of the GPU parity tests for f32 programs.

Three distances are always computed and printed (and appended to the file ACCY_B200_PARITY_REPORT
names, when set): GPU against the reference-order f32 oracle, GPU against the f64 evaluation, and
the reference-order oracle against f64.  The reference's serial f32 folds carry a rounding error
of their own (about sqrt(n) * eps), so the GPU's tree-shaped folds are held to

    |gpu - f64| <= tol + |ref - f64|          (at least as close to the exact result as the
                                                reference itself, up to the stated tolerance)
    |gpu - ref| <= tol + 2 * |ref - f64|      (which the first bound implies through f64)

with tol = 1e-5 relative for f32 (1e-12 for f64 programs).  "Relative" is against
max(|exact|, floor_frac * max|exact|): elements that cancel to nearly zero are measured against
the output's own scale.
"""
import os

import numpy as np


def rel_err(got, want, floor_frac):
    want = np.asarray(want, np.float64).reshape(-1)
    got = np.asarray(got, np.float64).reshape(-1)
    if want.size == 0:
        return 0.0
    floor = max(float(np.abs(want).max()) * floor_frac, 1e-30)
    return float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))


def check_three_distances(label, got, ref, exact, floor_frac, tol=1e-5):
    gpu_ref = rel_err(got, ref, floor_frac)
    gpu_f64 = rel_err(got, exact, floor_frac)
    ref_f64 = rel_err(ref, exact, floor_frac)
    line = "%s: |gpu-ref_order| %.3g  |gpu-f64| %.3g  |ref_order-f64| %.3g  (tol %g, floor %g of max)" % (
        label, gpu_ref, gpu_f64, ref_f64, tol, floor_frac)
    print(line)
    path = os.environ.get("ACCY_B200_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")
    assert gpu_f64 < tol + ref_f64, line
    assert gpu_ref < tol + 2.0 * ref_f64, line
    return gpu_ref, gpu_f64, ref_f64
