"""A projection y = x W^T + b with W held [out][in] row-major (src/graph/ops.rs:132-136).

Which kernel runs depends only on the precisions: float32 anywhere means the FP32-pipe
product (true 32-bit, no tensor-core mode); bfloat16 activations with bfloat16 weights go
to the tensor-core kernels.  A weight the checkpoint stores in 32-bit stays float32 even
in the bfloat16 engine and is multiplied on the FP32 pipe.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..kernels import api as K


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("a projection's weight must be [out, in]")
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self._fast = None

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        """``out`` (+)= x W^T + b.  ``accumulate`` adds into a float32 ``out``."""
        if x.shape[-1] != self.in_features:
            raise K.KernelError(
                f"projection takes width {self.in_features}, got {x.shape[-1]}")
        if out is None:
            if accumulate:
                raise ValueError("accumulate needs an output to add into")
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        if x.shape[0] == 0:
            return out
        if x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from ..kernels import gemm
            gemm.gemm_bf16(x, self.weight, self.bias, out, accumulate)
        else:
            K.gemm_simt(x, self.weight, self.bias, out, accumulate)
        return out

    def partial_sums(self, x: torch.Tensor):
        """If the tensor-core kernel would split this product along K (few tokens, few output
        rows), runs the splits and returns them as a ``Pending`` (bias included) for the next
        kernel to add; otherwise returns None and the caller uses ``forward``."""
        from ..kernels import gemm
        from .base import Pending
        if (x.dtype != torch.bfloat16 or self.weight.dtype != torch.bfloat16 or x.shape[0] == 0
                or not gemm.use_tensor_cores()):
            return None
        partial = K.gemm_tc_partial_sums(x, self.weight, gemm.status_word(x.device))
        return None if partial is None else Pending(partial, self.bias)
