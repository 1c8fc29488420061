"""Pre-norm block with two residual adds: h += mixer(norm1(h)); h += ffn(norm2(h))
(src/models/qwen2/graph.rs:59-64, 137, 154-155, 176)."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.base import LayerSpec
from .base import Block, CallBinding, StepContext


class PreNormBlock(Block):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def __init__(self, layer: LayerSpec):
        from ..registry import build_part
        self.prefix = layer.prefix
        self.mixer_norm = build_part("norm", layer.mixer_norm)
        self.mixer = build_part("mixer", layer.mixer)
        self.feed_forward_norm = build_part("norm", layer.feed_forward_norm)
        self.feed_forward = build_part("feed_forward", layer.feed_forward)

    def parts(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def tensor_specs(self, prefix: str = "") -> List:
        specs = []
        for part in self.parts():
            specs += part.tensor_specs(self.prefix)
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(self.prefix, weights)

    def export(self, prefix: str = "") -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {}
        for part in self.parts():
            out.update(part.export(self.prefix))
        return out

    accepts_pending = True     # its norms add a pending projection output while reading h

    @staticmethod
    def _normed(norm, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        pending = ctx.extras.pop("pending", None)
        if pending is not None:
            return norm.forward_settling(h, pending, ctx.act_dtype)
        return norm.forward(h, ctx.act_dtype)

    def mix(self, h: torch.Tensor, ctx: StepContext, binding: CallBinding) -> None:
        x = self._normed(self.mixer_norm, h, ctx)
        self.mixer.forward_add(x, ctx, binding, h)

    def feed(self, h: torch.Tensor, ctx: StepContext) -> None:
        x = self._normed(self.feed_forward_norm, h, ctx)
        self.feed_forward.forward_add(x, ctx, h)
