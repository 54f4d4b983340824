"""Rotary position encoding, rotate-half layout.

Frequencies as the reference builds them, in float32
(crates/synaptix-ops/src/pos/rope_cache.rs:16-38): ``f_i = theta^(-(2 i)/d)``,
angle ``= position * f_i``.  Rotation (crates/synaptix-ops/src/pos/rope.rs:84-100):
for ``i < d/2``: ``o[i] = x[i] cos - x[i+d/2] sin``, ``o[i+d/2] = x[i] sin + x[i+d/2] cos``;
elements at and above ``rotary_dim`` pass through.

The reference tabulates cos and sin per position (and casts the tables to the
compute dtype on its graph path, model.rs:1404-1407); here the kernel computes
the angle, sine and cosine in float32 from the position, so there is no table
capacity and no rounding of the table.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import PositionEncoding, Runtime


def rotary_inv_freq(theta: float, rotary_dim: int) -> np.ndarray:
    """``theta^(-(2i)/rotary_dim)`` for ``i < rotary_dim/2``, computed in float32."""
    i = np.arange(rotary_dim // 2, dtype=np.float32)
    exponent = -(np.float32(2.0) * i) / np.float32(rotary_dim)
    return np.power(np.float32(theta), exponent).astype(np.float32)


# one device tensor per (theta, rotary_dim, device): layers with the same rotation share it, and what a step derives
# from it (a table of cosines and sines) is made once a step, not once a layer
_INV_FREQ = {}


class RotaryHalf(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None):
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.theta = float(theta)
        self.inv_freq = None

    def bind(self, tensors, rt: Runtime) -> None:
        key = (self.theta, self.rotary_dim, str(rt.device))
        if key not in _INV_FREQ:
            _INV_FREQ[key] = torch.from_numpy(rotary_inv_freq(self.theta, self.rotary_dim)).to(rt.device)
        self.inv_freq = _INV_FREQ[key]

    def rotation(self):
        return self.inv_freq, self.rotary_dim


class NoPosition(PositionEncoding):
    """Queries and keys are used as they are."""
