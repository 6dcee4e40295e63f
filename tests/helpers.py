"""Shared checks for the parity tests."""
from __future__ import annotations

import numpy as np

# The reference's own tolerance for the Q8 path (tests/q4k_q8_test.cpp:129):
REF_ABS, REF_REL = 0.02, 0.002
# The benchmark contract: max relative error 2e-3 and mean absolute error <= 1e-4 * ||row||,
# "row" being one token's output vector.  Relative error is taken against |ref| floored at
# 1e-3 of the row's rms, so that outputs that cancel to ~0 do not divide by ~0.
MAX_REL, MAE_ROW = 2e-3, 1e-4


def assert_close_reference(y: np.ndarray, ref: np.ndarray) -> None:
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert np.isfinite(y).all()
    err = np.abs(y - ref)
    bad = err > REF_ABS + REF_REL * np.abs(ref)
    assert not bad.any(), f"{bad.sum()} outputs outside 0.02+0.002|ref|, worst {err.max()}"


def assert_close_contract(y: np.ndarray, ref: np.ndarray) -> None:
    """y, ref: [tokens, rows]."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert np.isfinite(y).all()
    err = np.abs(y - ref)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    rel = err / np.maximum(np.abs(ref), 1e-3 * rms + 1e-30)
    assert rel.max() <= MAX_REL, f"max relative error {rel.max():.3e} > {MAX_REL}"
    norm = np.sqrt((ref ** 2).sum(axis=1))
    mae = err.mean(axis=1)
    assert (mae <= MAE_ROW * norm + 1e-30).all(), f"MAE {mae.max():.3e} vs 1e-4*||row|| {MAE_ROW * norm.min():.3e}"
