"""Seeded synthetic inputs: one PCG64 stream per key, so every caller that names the same key draws the same
numbers (parameter initialisation of the training executor, the benchmark's operands and batches, the tests).

The distributions are the ones the reference draws at start-up — He-normal filters and dense weights
(seann/operands/seblas/Conv2D.cu:45-50, Linear.cu:42-46) — with fixed seeds in place of its clock seeding.
"""
from __future__ import annotations

import zlib

import numpy as np


def rng_for(*key) -> np.random.Generator:
    seed = zlib.crc32(repr(key).encode())
    return np.random.Generator(np.random.PCG64(seed))


def uniform_pm1(shape, *key) -> np.ndarray:
    return rng_for("u", *key).uniform(-1.0, 1.0, size=shape).astype(np.float32)


def normal(shape, *key, std: float = 1.0) -> np.ndarray:
    return (rng_for("n", *key).standard_normal(size=shape) * std).astype(np.float32)


def he_normal_filter(oc: int, ic: int, fh: int, fw: int, *key) -> np.ndarray:
    """He-normal filter N(0, 2/(IC*FH*FW))."""
    return normal((oc, ic, fh, fw), "he", *key, std=float(np.sqrt(2.0 / (ic * fh * fw))))
