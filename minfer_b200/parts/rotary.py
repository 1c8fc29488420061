"""Rotary position encoding: pairs of a head's dimensions are rotated by
``pos * frequency_scale / theta^(2i/rotary_dim)``.

The reference (src/graph/cpu_backend.rs:403-434) rotates the whole head, pairs
``(i, i + hd/2)`` for its ``NonInterleaved`` style (Qwen2, src/models/qwen2/loader.rs:144)
or ``(2i, 2i+1)`` for ``Interleaved`` (src/vec_ops.rs:6-14).  The reference forms the angle
``pos * freq`` in float32, which is off by about 1e-4 rad at position 2,000; here the inverse
frequencies are kept in float64, the angle is formed and reduced modulo 2 pi in float64 on the
device, and its sine and cosine are float32.
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
        return self.frequency_scale / torch.pow(
            torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.rotary_dim)

    def fused_rotary(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int, int]]:
        key = str(device)
        if key not in self._inv_freq:
            self._inv_freq[key] = self.inverse_frequencies().to(device)
        return self._inv_freq[key], self.rotary_dim, STYLES[self.style]


class NoPosition(PositionEncoding):
    """No position encoding at all: queries and keys pass through."""

    def fused_rotary(self, device: torch.device):
        return None, 0, 0
