"""Shared helpers for the parity tests."""
import numpy as np

REL_TOL = 1e-3  # bar stated for f32 outputs: max|y - y_ref| / max|y_ref| <= 1e-3


def rel_err(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.abs(ref).max()
    return float(np.abs(y - ref).max() / (denom if denom > 0 else 1.0))


def make_case(seed, n, k, m, w_std=0.02):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * w_std).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    return w, x
