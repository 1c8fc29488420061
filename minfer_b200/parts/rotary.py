"""Rotary position encoding: pairs of a head's dimensions are rotated by
``pos * frequency_scale / theta^(2i/rotary_dim)``.

The reference (src/graph/cpu_backend.rs:403-434) rotates the whole head, pairs
``(i, i + hd/2)`` for its ``NonInterleaved`` style (Qwen2, src/models/qwen2/loader.rs:144)
or ``(2i, 2i+1)`` for ``Interleaved`` (src/vec_ops.rs:6-14).  The inverse frequencies are
made once in float64 and rounded to float32; the angle and its sine and cosine are float32
on the device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import PositionEncoding

STYLES = {"neox": 0, "interleaved": 1}


class Rotary(PositionEncoding):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def __init__(self, head_dim: int, rotary_dim: int, theta: float, frequency_scale: float = 1.0,
                 style: str = "neox"):
        if style not in STYLES:
            raise ValueError(f"rotary style must be one of {sorted(STYLES)}, got {style!r}")
        if rotary_dim % 2 != 0 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and in (0, head_dim={head_dim}]")
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim)
        self.theta = float(theta)
        self.frequency_scale = float(frequency_scale)
        self.style = style
        self._inv_freq: dict = {}

    def inverse_frequencies(self) -> torch.Tensor:
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        return (self.frequency_scale / torch.pow(
            torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.rotary_dim)).to(torch.float32)

    def fused_rotary(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int, int]]:
        key = str(device)
        if key not in self._inv_freq:
            self._inv_freq[key] = self.inverse_frequencies().to(device)
        return self._inv_freq[key], self.rotary_dim, STYLES[self.style]


class NoPosition(PositionEncoding):
    """No position encoding at all: queries and keys pass through."""

    def fused_rotary(self, device: torch.device):
        return None, 0, 0
