"""Position encodings a mixer can be given.

A position part offers two things to the mixer that owns it: ``rotary_dim`` (how many
leading dims of each head are rotated; 0 = none) and ``inv_freq`` (float32,
``rotary_dim / 2`` entries).  The rotation itself happens in the mixer's kernel at each
row's absolute position, with the angle ``float32(p) * inv_freq[d]`` computed in
32-bit (model/Prim.cajeta:1917-1940).

``rope``: ``inv_freq[d] = theta^(-2d / rotary_dim)`` computed in float32 as the
reference does (model/Prim.cajeta:1866-1880; per-layer state, model/Attention.cajeta:72-99).
``none``: no rotation.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part


@register_part("position", "rope")
class RotaryEncoding(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.theta = float(spec["theta"])
        if self.rotary_dim % 2 != 0 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim must be even and within (0, head_dim={self.head_dim}], found {self.rotary_dim}")
        half = self.rotary_dim // 2
        d = np.arange(half, dtype=np.float32)
        exponent = (np.float32(0.0) - np.float32(2.0) * d) / np.float32(self.rotary_dim)
        inv = np.power(np.float32(self.theta), exponent).astype(np.float32)
        self.inv_freq = torch.from_numpy(inv).to(runtime.device)


@register_part("position", "none")
class NoPosition(Part):
    def __init__(self, spec, prefix, runtime):
        super().__init__(spec, prefix, runtime)
        self.rotary_dim = 0
        self.inv_freq = None
