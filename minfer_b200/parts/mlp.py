"""Gated feed-forward: down( act(gate(x)) * up(x) ), no biases.

The reference builds it as silu + mul that its fusion pass folds into SwiGLU
(src/models/qwen2/graph.rs:154-175, src/graph/fusion.rs:37-87), with
silu(z) = z / (1 + exp(-z)) (src/vec_ops.rs:131-146); its Metal path packs gate|up into
one matrix (src/models/qwen2/graph.rs:148-169).  Here gate|up is always one product and
the down projection adds into the residual stream in its epilogue.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import api as K
from ..weights.spec import MATRIX, Init, TensorSpec
from .base import FeedForward, StepContext, settle_pending
from .linear import Linear


class GatedMlp(FeedForward):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        return ["ops", "gemm_tc"] if dtype == torch.bfloat16 else ["ops", "gemm_simt"]

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 init_std: float = 0.02):
        if activation != "silu":
            raise ValueError(f"the gated feed-forward has the 'silu' activation only, got "
                             f"{activation!r}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.init_std = float(init_std)
        self.interleaved = False
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}mlp."
        init = Init(0.0, self.init_std)
        return [TensorSpec(f"{p}gate_proj.weight", (self.intermediate_size, self.hidden_size),
                           MATRIX, init),
                TensorSpec(f"{p}up_proj.weight", (self.intermediate_size, self.hidden_size),
                           MATRIX, init),
                TensorSpec(f"{p}down_proj.weight", (self.hidden_size, self.intermediate_size),
                           MATRIX, init)]

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}mlp."
        g, u = weights[f"{p}gate_proj.weight"], weights[f"{p}up_proj.weight"]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        # bfloat16: rows alternate gate, up so that the tensor-core kernel's epilogue finds a
        # pair in neighbouring lanes and writes silu(gate) * up directly; float32: gates first
        self.interleaved = g.dtype == torch.bfloat16
        if self.interleaved:
            packed = torch.stack([g, u], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            packed = torch.cat([g, u], dim=0)
        self.gate_up = Linear(packed.contiguous())
        self.down = Linear(weights[f"{p}down_proj.weight"])
        self.accepts_row_scale = self.interleaved and self.gate_up.takes_row_scale()

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}mlp."
        w = self.gate_up.weight
        if self.interleaved:
            pairs = w.view(self.intermediate_size, 2, self.hidden_size)
            gate, up = pairs[:, 0], pairs[:, 1]
        else:
            gate, up = w[:self.intermediate_size], w[self.intermediate_size:]
        return {f"{p}gate_proj.weight": gate, f"{p}up_proj.weight": up,
                f"{p}down_proj.weight": self.down.weight}

    def forward_add(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        from ..kernels import gemm
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=ctx.act_dtype,
                          device=x.device)
        w = self.gate_up.weight
        rs = ctx.input_scale                       # the norm's 1/rms, if this product is to apply it
        if (self.interleaved and x.shape[0] > 0 and gemm.use_tensor_cores()
                and K.gemm_tc_supported(x, w)):
            if rs is not None:
                K.gemm_tc_fused(x, w, None, act, K.EPI_SWIGLU, gemm.status_word(x.device), row_scale=rs)
            else:
                K.gemm_tc(x, w, None, act, K.EPI_SWIGLU, gemm.status_word(x.device))
        else:
            if rs is not None:
                raise K.KernelError("a row scale needs the tensor-core product")
            gu = self.gate_up.forward(x, ctx.act_dtype)
            K.swiglu(gu, act, self.interleaved)
        target = ctx.extras.pop("prepare_for", None)
        if target is not None:
            settle_pending(ctx, residual)
            prepared = self.down.accumulate_prepared(act, residual, target)
            if prepared is not None:
                ctx.extras["prepared"] = prepared
                return
        pending = self.down.partial_sums(act)
        if pending is None:
            self.down.forward(act, torch.float32, out=residual, accumulate=True)
        else:
            settle_pending(ctx, residual)          # never two at once
            ctx.extras["pending"] = pending
