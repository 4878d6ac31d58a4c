"""Rotary position encoding: the table of inverse frequencies a mixer rotates q and k with.

inv_i = theta^(-2i/hd); with llama3 scaling, frequencies whose wavelength exceeds
original_max/low_freq_factor are divided by `factor`, those below original_max/high_freq_factor
are kept, and the band between is blended (crates/engine/src/backend/cpu/rope.rs:36-61). The
table is float32 and every step after the power is taken in float32, as there; the power itself
is computed in float64 and rounded. The rotation (rotate-half pairing, angle = float32(position)
* inv_i) happens in the mixer's kernel.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .base import PositionEncoding


def rotary_inv_freq(head_dim: int, theta: float, scaling=None) -> np.ndarray:
    f32 = np.float32
    half = head_dim // 2
    inv = np.empty(half, dtype=f32)
    for i in range(half):
        expo = f32(2 * i) / f32(head_dim)
        inv[i] = f32(1.0) / f32(math.pow(float(theta), float(expo)))
    if scaling is None:
        return inv
    factor, low, high = f32(scaling.factor), f32(scaling.low_freq_factor), f32(scaling.high_freq_factor)
    old_ctx = f32(scaling.original_max_position_embeddings)
    low_freq_wavelen = old_ctx / low
    high_freq_wavelen = old_ctx / high
    two_pi = f32(2.0) * f32(math.pi)
    out = np.empty_like(inv)
    for i in range(half):
        v = inv[i]
        wavelen = two_pi / v
        if wavelen < high_freq_wavelen:
            out[i] = v
        elif wavelen > low_freq_wavelen:
            out[i] = v / factor
        else:
            smooth = (old_ctx / wavelen - low) / (high - low)
            out[i] = (f32(1.0) - smooth) * v / factor + smooth * v
    return out


class Rotary(PositionEncoding):
    """theta and the scaling rule are parameters; `inv_freq` is the device table [head_dim/2]."""

    def __init__(self, head_dim: int, theta: float, scaling=None, device="cuda"):
        if head_dim % 2 != 0:
            raise ValueError(f"rotary positions need an even head_dim, got {head_dim}")
        self.head_dim = head_dim
        self.theta = float(theta)
        self.scaling = scaling
        self.inv_freq_host = rotary_inv_freq(head_dim, theta, scaling)
        self.inv_freq = torch.from_numpy(self.inv_freq_host.copy()).to(device)
