"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, the weight applied after the scale, no bias
(src/vec_ops.rs:500-522; src/graph/cpu_backend.rs:195-213)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import VECTOR, Init, TensorSpec
from .base import Norm


class RmsNorm(Norm):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops"]

    def __init__(self, size: int, eps: float, name: str = "norm", init_std: float = 0.0):
        self.size = int(size)
        self.eps = float(eps)
        self.name = name
        self.init_std = float(init_std)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return [TensorSpec(f"{prefix}{self.name}.weight", (self.size,), VECTOR,
                           Init(1.0, self.init_std))]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        self.weight = weights[f"{prefix}{self.name}.weight"]

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        return {f"{prefix}{self.name}.weight": self.weight}

    def foldable(self):
        return (self.weight, self.eps, self.size)

    def forward(self, x32: torch.Tensor, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x32.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype, device=x32.device)
        K.rmsnorm(x32, self.weight, self.eps, out, rows)
        return out

    def forward_settling(self, h: torch.Tensor, pending, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((h.shape[0], self.size), dtype=out_dtype, device=h.device)
        K.add_rmsnorm(h, pending.partial, pending.partial.shape[0], pending.bias, self.weight,
                      self.eps, out)
        return out
