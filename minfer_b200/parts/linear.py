"""A projection y = x W^T + b with W held [out][in] row-major (src/graph/ops.rs:132-136).

Which kernel runs depends only on the precisions: float32 anywhere means the FP32-pipe
product (true 32-bit, no tensor-core mode); bfloat16 activations with bfloat16 weights go
to the tensor-core kernels.  A weight the checkpoint stores in 32-bit stays float32 even
in the bfloat16 engine and is multiplied on the FP32 pipe.
"""
from __future__ import annotations

from typing import Optional

import torch

import os

from ..kernels import api as K

# MINFER_B200_FOLD_NORMS=0: every norm runs as a kernel of its own (for comparison)
FOLD_NORMS = os.environ.get("MINFER_B200_FOLD_NORMS", "1") != "0"


class Linear:
    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        if weight.dim() != 2:
            raise ValueError("a projection's weight must be [out, in]")
        self.weight = weight
        self.bias = bias
        self.out_features, self.in_features = weight.shape
        self._fast = None

    def takes_row_scale(self) -> bool:
        """The tensor-core kernel multiplies this projection (only it can apply a row scale)."""
        from ..kernels import gemm
        w = self.weight
        return (w.dtype == torch.bfloat16 and gemm.use_tensor_cores() and w.shape[1] % 8 == 0
                and w.stride(1) == 1 and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype,
                out: Optional[torch.Tensor] = None, accumulate: bool = False,
                row_scale=None) -> torch.Tensor:
        """``out`` (+)= x W^T + b.  ``accumulate`` adds into a float32 ``out``.  ``row_scale``
        (a ``RowScale``): the rows of ``x`` still lack their norm's 1/rms; the kernel applies it."""
        if x.shape[-1] != self.in_features:
            raise K.KernelError(
                f"projection takes width {self.in_features}, got {x.shape[-1]}")
        if out is None:
            if accumulate:
                raise ValueError("accumulate needs an output to add into")
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype, device=x.device)
        if x.shape[0] == 0:
            return out
        if row_scale is not None:
            from ..kernels import gemm
            if not (self.takes_row_scale() and K.gemm_tc_supported(x, self.weight)):
                raise K.KernelError("a row scale needs the tensor-core product")
            K.gemm_tc_fused(x, self.weight, self.bias, out, K.EPI_ACCUM if accumulate else K.EPI_STORE,
                            gemm.status_word(x.device), row_scale=row_scale)
            return out
        if x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            from ..kernels import gemm
            gemm.gemm_bf16(x, self.weight, self.bias, out, accumulate)
        else:
            K.gemm_simt(x, self.weight, self.bias, out, accumulate)
        return out

    def partial_sums(self, x: torch.Tensor, row_scale=None):
        """If the tensor-core kernel would split this product along K (few tokens, few output
        rows), runs the splits and returns them as a ``Pending`` (bias included) for the next
        kernel to add; otherwise returns None and the caller uses ``forward``."""
        from ..kernels import gemm
        from .base import Pending
        if (x.dtype != torch.bfloat16 or self.weight.dtype != torch.bfloat16 or x.shape[0] == 0
                or not gemm.use_tensor_cores()):
            return None
        if row_scale is not None:
            if not K.gemm_tc_supported(x, self.weight):
                return None
            partial = K.gemm_tc_fused(x, self.weight, None, None, K.EPI_STORE,
                                      gemm.status_word(x.device), row_scale=row_scale, defer=True)
        else:
            partial = K.gemm_tc_partial_sums(x, self.weight, gemm.status_word(x.device))
        return None if partial is None else Pending(partial, self.bias)

    def accumulate_prepared(self, x: torch.Tensor, residual: torch.Tensor, norm):
        """``residual`` += x W^T + b, complete when the call returns, together with what ``norm``
        (which reads ``residual`` next) needs: returns a ``Prepared``, or None (and does nothing)
        if ``norm`` is not foldable or no kernel does this at these sizes."""
        from ..kernels import gemm
        from .base import Prepared
        fold = norm.foldable() if norm is not None else None
        m = x.shape[0]
        if (fold is None or m == 0 or x.dtype != torch.bfloat16 or not self.takes_row_scale()
                or not K.gemm_tc_supported(x, self.weight) or residual.dtype != torch.float32
                or not residual.is_contiguous() or not FOLD_NORMS):
            return None
        weight, eps, size = fold
        if size != self.out_features or weight.dtype != torch.float32:
            return None
        parts = K.gemm_tc_prep_parts(m, self.out_features, self.in_features)
        if parts == 0:
            return None
        xp = torch.empty((m, self.out_features), dtype=torch.bfloat16, device=x.device)
        ssq = torch.empty((parts, m), dtype=torch.float32, device=x.device)
        K.gemm_tc_fused(x, self.weight, self.bias, residual, K.EPI_ACCUM, gemm.status_word(x.device),
                        prep_x=xp, prep_weight=weight, prep_ssq=ssq)
        return Prepared(xp, K.RowScale(ssq, size, eps), norm)
