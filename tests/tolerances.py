"""Tolerances of the comparisons with the plain implementation, fixed before
the engine was measured against them and not to be widened to pass.

A bound is relative to the size of the reference logits: atol = k * (1 + max|ref|).
32-bit path: sums of a few thousand 32-bit products reordered, k = 4e-6 (a few
dozen units of 32-bit rounding). bfloat16 path: weights are exact but every
activation between kernels and every cached key and value is rounded to 8 bits
of mantissa (2^-9 relative each), through up to six layers: k = 3e-2.
Two bfloat16 runs that differ only in how the work was cut go through the same
roundings except where another kernel serves the shape: k = 2e-2.
Deeper models: the roundings of the layers are independent, so their sum grows
with the square root of their number; for more than six layers both bounds
against the plain implementation are multiplied by sqrt(layers / 6)
(`k_for_depth`; sixteen layers: 1.63 times). The bounds between two cuttings
of the same run stay as they are.
"""
import numpy as np

K = {"float32": 4e-6, "bfloat16": 3e-2}
K_SELF = {"float32": 1e-6, "bfloat16": 2e-2}


def k_for_depth(dtype, layers):
    return K[dtype] * max(1.0, layers / 6.0) ** 0.5


def check_close(got, ref, dtype, what="", k=None):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    tol = (K[dtype] if k is None else k) * (1.0 + np.abs(ref).max())
    err = np.abs(got - ref)
    if err.max() > tol:
        i = np.unravel_index(err.argmax(), err.shape)
        first = int(np.argmax((err > tol).any(axis=-1))) if err.ndim > 1 else int(np.argmax(err > tol))
        raise AssertionError(f"{what}: max |err| {err.max():.3e} > {tol:.3e} at {i}; first bad row {first}")
    return err.max()
