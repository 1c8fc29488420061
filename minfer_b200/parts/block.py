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

    def entry_norm(self):
        if self.mixer_norm.foldable() is not None and getattr(self.mixer, "accepts_row_scale", False):
            return self.mixer_norm
        return None

    @staticmethod
    def _normed(norm, h: torch.Tensor, ctx: StepContext, consumer):
        """The norm's output for ``consumer``, as (x, row scale): a prepared input if the product
        before left one for this very norm and the consumer can apply the scale, else the norm
        as a kernel (which also adds a pending projection output into ``h``)."""
        prepared = ctx.extras.pop("prepared", None)
        if (prepared is not None and prepared.norm is norm
                and getattr(consumer, "accepts_row_scale", False)):
            return prepared.x, prepared.scale
        pending = ctx.extras.pop("pending", None)
        if pending is not None:
            return norm.forward_settling(h, pending, ctx.act_dtype), None
        return norm.forward(h, ctx.act_dtype), None

    def _call(self, part, x, scale, ctx, target, *args) -> None:
        ctx.input_scale = scale
        if target is not None and getattr(part, "accepts_row_scale", False):
            ctx.extras["prepare_for"] = target
        try:
            part.forward_add(x, ctx, *args)
        finally:
            ctx.input_scale = None
            ctx.extras.pop("prepare_for", None)

    def mix(self, h: torch.Tensor, ctx: StepContext, binding: CallBinding) -> None:
        x, scale = self._normed(self.mixer_norm, h, ctx, self.mixer)
        # the mixer's last product may prepare the input of the norm before the feed-forward,
        # unless the engine drops rows of h between the two
        target = None
        if (ctx.extras.get("rows_stay", True) and self.feed_forward_norm.foldable() is not None
                and getattr(self.feed_forward, "accepts_row_scale", False)):
            target = self.feed_forward_norm
        self._call(self.mixer, x, scale, ctx, target, binding, h)

    def feed(self, h: torch.Tensor, ctx: StepContext) -> None:
        x, scale = self._normed(self.feed_forward_norm, h, ctx, self.feed_forward)
        # the feed-forward's last product may prepare the input of the norm that reads h next
        # (the next block's first, or the model's last), which the engine names
        self._call(self.feed_forward, x, scale, ctx, ctx.extras.get("next_norm"), h)
