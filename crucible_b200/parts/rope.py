"""Rotary position encoding with half-split pairing.

inv_freq_i = theta^(-2i/rotary_dim); angle = position * inv_freq_i;
out[i] = x[i]*cos - x[i+r/2]*sin; out[i+r/2] = x[i]*sin + x[i+r/2]*cos
(`model.py:131-145`; the engine builds the tables in f64 and stores f32,
`engine/src/ops.rs:101-115`; kernel `engine/kernels/kernels.cu:1677-1706`).
The tables are fp32 in both engine dtypes and the rotation is fp32 arithmetic.
"""
from __future__ import annotations

import torch

from ..config.model_config import PositionSpec
from .base import POSITIONS, PositionEncoding


_TABLES = {}     # (theta, rotary_dim, positions, device) -> (cos, sin), read-only


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2 != 0 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be a positive even number, got {spec.rotary_dim}")
        self.spec = spec
        self.cos = None
        self.sin = None

    def bind(self, tensors, dtype, device):
        # layers with the same rotation share one pair of tables (a model of 32 layers
        # with 131,072 positions would otherwise hold 32 identical pairs of 33 MB)
        key = (float(self.spec.theta), self.spec.rotary_dim, self.spec.max_positions,
               str(torch.device(device)))
        hit = _TABLES.get(key)
        if hit is None:
            half = self.spec.rotary_dim // 2
            i = torch.arange(half, dtype=torch.float64)
            inv_freq = torch.pow(torch.tensor(self.spec.theta, dtype=torch.float64),
                                 -2.0 * i / self.spec.rotary_dim)
            pos = torch.arange(self.spec.max_positions, dtype=torch.float64)
            ang = torch.outer(pos, inv_freq)
            hit = (ang.cos().to(torch.float32).contiguous().to(device),
                   ang.sin().to(torch.float32).contiguous().to(device))
            if len(_TABLES) >= 8:
                _TABLES.pop(next(iter(_TABLES)))
            _TABLES[key] = hit
        self.cos, self.sin = hit

    def rotation(self):
        return self.cos, self.sin, self.spec.rotary_dim


POSITIONS.register("rope", RotaryEncoding)
