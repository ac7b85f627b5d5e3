"""Seeded synthetic tensors.

Every tensor is drawn from its own counter-based Philox stream keyed by (seed, tensor id), so the
same (seed, id, shape) gives the same bits on any machine and in any order of generation.
"""
from __future__ import annotations

import zlib

import numpy as np


def _rng(seed: int, tensor_id) -> np.random.Generator:
    if isinstance(tensor_id, str):
        tensor_id = zlib.crc32(tensor_id.encode())
    return np.random.Generator(np.random.Philox(key=[int(seed) & (2**64 - 1), int(tensor_id) & (2**64 - 1)]))


def normal(seed, tensor_id, shape, mean=0.0, std=1.0) -> np.ndarray:
    return (_rng(seed, tensor_id).standard_normal(shape, dtype=np.float32) * np.float32(std)
            + np.float32(mean)).astype(np.float32)


def uniform(seed, tensor_id, shape, lo=0.0, hi=1.0) -> np.ndarray:
    r = _rng(seed, tensor_id).random(shape, dtype=np.float32)
    return (r * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def bn_params(seed, tensor_id, channels):
    """gamma U(0.5,1.5), beta N(0,0.1), running mean N(0,0.1), running var U(0.5,1.5)."""
    base = tensor_id if isinstance(tensor_id, str) else str(tensor_id)
    return (uniform(seed, base + "/gamma", channels, 0.5, 1.5), normal(seed, base + "/beta", channels, 0.0, 0.1),
            normal(seed, base + "/mean", channels, 0.0, 0.1), uniform(seed, base + "/var", channels, 0.5, 1.5))
