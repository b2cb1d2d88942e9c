"""Rotary position encoding: the table of inverse frequencies.

spec options: theta, head_dim, rotary_dim (defaults to head_dim; 0: nothing turns), exact_table (the table worked
out in 64-bit and rounded once), frequency_divisor (every frequency is divided by it: positions stretched by that
factor; absent: as they are), pairing ('half', the default: element j
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
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim or self.rotary_dim < 0:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        if spec.options.get("exact_table", False):
            # every frequency is the 32-bit number nearest to theta^(-2j / rotary_dim): worked out in 64-bit, rounded once
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / max(1, self.rotary_dim)
            self.inv_freq = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -exponent).to(torch.float32)
        else:
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / max(1, self.rotary_dim)
            self.inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32)
        divisor = spec.options.get("frequency_divisor")
        if divisor is not None:
            if not float(divisor) > 0:
                raise ValueError(f"frequency_divisor {divisor!r} must be positive")
            # theta^(-2j / rotary_dim) / divisor in 64-bit, rounded once
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float64) / max(1, self.rotary_dim)
            exact = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -exponent) / float(divisor)
            self.inv_freq = exact.to(torch.float32) if spec.options.get("exact_table", False) else self.inv_freq / float(divisor)
        if device is not None:
            self.inv_freq = self.inv_freq.to(device)

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self
