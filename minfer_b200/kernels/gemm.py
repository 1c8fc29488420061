"""Chooses the kernel of a bfloat16 x bfloat16 projection."""
from __future__ import annotations

from typing import Any, Optional

import torch

from . import api as K


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
              out: torch.Tensor, accumulate: bool, owner: Any = None) -> None:
    K.gemm_simt(x, weight, bias, out, accumulate)
