"""Seeded synthetic inputs for the attention path.

Every tensor comes from its own numpy stream keyed by (seed, config id, layer,
tensor id), drawn N(0, 1) in float32 and cast to f16, so that a test, the
benchmark and the CPU baseline can regenerate the same bytes independently.
Tensor ids: 0 q, 1 k_new, 2 v_new, 3 K_past, 4 V_past.
"""
from __future__ import annotations

import numpy as np

T_Q, T_K_NEW, T_V_NEW, T_K_PAST, T_V_PAST = range(5)


def tensor(seed, cfg_id, layer, tensor_id, shape):
    rng = np.random.default_rng([seed, cfg_id, layer, tensor_id])
    return rng.standard_normal(shape, dtype=np.float32).astype(np.float16)


def ones_weight():
    """Norm weight of 1.0 for the 128 head dims (the configs use weight 1)."""
    return np.ones(128, dtype=np.float16)
