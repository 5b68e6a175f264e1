"""Rotary position encoding: the table of inverse frequencies.

spec options: theta, head_dim, rotary_dim (defaults to head_dim), pairing ('half', the default: element j
turns with j + rotary_dim/2, src/wllm/models/llama.py:47-49; 'interleaved': 2j with 2j + 1).  The table is
inv_freq[j] = theta^(-2j / rotary_dim) in 32-bit (src/wllm/models/llama.py:55) and
never leaves 32-bit; angles are position * inv_freq, computed in the kernel from the
token's absolute position, so no table length limits the context.  Pairs are
(j, j + rotary_dim/2) (src/wllm/models/llama.py:47-49).
"""
from __future__ import annotations

import torch

from .base import POSITIONS


@POSITIONS.register("rope")
class RotaryPosition:
    def __init__(self, spec, device=None):
        self.head_dim = int(spec.head_dim)
        self.rotary_dim = int(spec.options.get("rotary_dim", self.head_dim))
        self.theta = float(spec.theta)
        self.pairing = spec.options.get("pairing", "half")
        if self.pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {self.pairing!r}: 'half' or 'interleaved'")
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32)
        if device is not None:
            self.inv_freq = self.inv_freq.to(device)

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self
