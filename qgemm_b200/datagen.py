"""Seeded synthetic operands with the value distributions of the benchmark configurations.

The reference's harness fills operands from a closed-form pattern and ignores its seed
(tests/includes/test_config.h:230,251-258); the configurations measured here ask for seeded random
data instead. One counter-based generator (numpy Philox) keyed by (seed, stream) produces every
operand, so a test, the benchmark and a CPU check all see the same bits for the same seed.
"""
from __future__ import annotations

import numpy as np


def _rng(seed: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[int(seed), int(stream)]))


def uniform(shape, seed: int, stream: int = 0, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    """float32 uniform [lo, hi)."""
    r = _rng(seed, stream).random(shape, dtype=np.float32)
    return (lo + (hi - lo) * r).astype(np.float32)


def normal(shape, seed: int, stream: int = 0) -> np.ndarray:
    """float32 standard normal."""
    return _rng(seed, stream).standard_normal(shape, dtype=np.float32)


def int8_uniform(shape, seed: int, stream: int = 0) -> np.ndarray:
    """int8 uniform integers in [-127, 127]."""
    return _rng(seed, stream).integers(-127, 128, size=shape, dtype=np.int8)


def scale_pair(seed: int, stream: int = 99):
    """Two per-matrix quantisation coefficients, float32 uniform [1e-3, 1e-2)."""
    r = _rng(seed, stream).random(2, dtype=np.float32)
    s = (np.float32(1e-3) + np.float32(9e-3) * r).astype(np.float32)
    return np.float32(s[0]), np.float32(s[1])
