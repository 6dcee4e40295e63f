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


def fitter_cases(seed: int, random_blocks: int) -> np.ndarray:
    """Seeded float32 [blocks, 256] inputs for the Q4_K fitter: the corner cases of
    src/compiler/quantization/q4k.cpp:186-278 first (constant and one-sided groups, groups whose
    six-bit scale rounds to zero, fp16-subnormal and overflowing block scales, every refusal),
    then `random_blocks` blocks of mixed scale and tail weight."""
    rng = np.random.default_rng(seed)
    f32 = np.float32
    rows = []
    add = lambda a: rows.append(np.asarray(a, dtype=f32).reshape(256))
    normal = lambda s: rng.standard_normal(256) * s
    add(normal(0.02))                                     # typical weights
    add(np.zeros(256))                                    # all zero
    add(np.full(256, 0.5))                                # constant, positive
    add(np.full(256, -0.75))                              # constant, negative: max == min
    add(rng.uniform(0.1, 1.0, 256))                       # one-sided positive
    add(-rng.uniform(0.1, 1.0, 256))                      # one-sided negative
    w = normal(0.01); w[64:96] *= 2000.0; add(w)          # one dominant group: others get scale 0
    w = normal(1.0); w[rng.random(256) < 0.3] = 0.0; w[5] = -0.0; w[32] = -0.0; add(w)
    add(normal(1e-30))                                    # block scale below fp16 subnormals
    add(normal(3e-7))                                     # block scale an fp16 subnormal
    add(normal(1e6))                                      # large but representable
    w = normal(0.02); w[:32] = np.linspace(-1, 1, 32); add(w)
    w = normal(0.02); w[96:128] = 0.125; add(w)           # a constant group inside a live block
    add(np.round(normal(3.0)))                            # many exact ties
    add(np.tile(np.arange(16, dtype=f32), 16) - 8.0)      # exactly representable grid
    w = np.zeros(256); w[200] = 1.0; add(w)               # a single spike
    add(-1000.0 + normal(1e-3))                           # narrow band far below zero: offset >> step
    add(1000.0 + normal(1e-3))                            # narrow band far above zero: minimum capped at 0
    w = normal(0.02); w[:32] = -50.0 + rng.standard_normal(32) * 1e-4; add(w)
    add(-np.tile(np.linspace(1.0, 2.0, 32), 8))           # one-sided ramps
    add(-np.abs(normal(1.0)) - 1e3 * np.repeat(rng.random(8), 32))
    # refusals
    add(normal(1e-38))                                    # fitting reciprocal overflow
    add(normal(2e-38) + 1e-37)                            # compression reciprocal overflow (or earlier)
    add(normal(1e8))                                      # fp16 scale overflow
    w = normal(1.0); w[77] = np.nan; add(w)
    w = normal(1.0); w[255] = np.inf; add(w)
    w = normal(1.0); w[0] = -np.inf; add(w)
    w = normal(1.0); w[130] = 2e10; add(w)
    w = normal(1.0); w[10] = -3e10; w[200] = np.nan; add(w)  # the first offender decides
    w = normal(1.0); w[10] = np.nan; w[9] = 3e10; add(w)
    scales = 10.0 ** rng.uniform(-4, 2, random_blocks)
    for i in range(random_blocks):
        kind = i % 4
        if kind == 0:
            w = rng.standard_normal(256)
        elif kind == 1:
            w = rng.standard_t(3, 256)
        elif kind == 2:
            w = rng.uniform(-1, 1, 256) * rng.uniform(0.01, 1, 8).repeat(32)
        else:  # bf16-representable, as weights arrive from a checkpoint
            w = (rng.standard_normal(256).astype(f32).view(np.uint32) & 0xFFFF0000).view(f32)
        add(w * scales[i])
    return np.stack(rows)
