"""Interfaces of the parts a layer is put together from, and what a part sees of a step.

A part has its sizes and constants as constructor parameters, names the tensors it wants
from the checkpoint, and runs on whatever batch the step context describes.  No part knows
which model it is in.  The five roles:

``Norm``               ``forward(x32, out_dtype, rows=None) -> y``
``PositionEncoding``   either ``fused_rotary()`` (parameters the fused rotary kernel takes)
                       or ``apply(qkv32, ctx, n_heads, n_kv_heads, head_dim)`` in place
``Mixer``              ``cache_request()``, ``state_request()``,
                       ``forward_add(x, ctx, binding, residual)``
``FeedForward``        ``forward_add(x, ctx, residual)``
``Block``              ``mix(h, ctx, binding)`` then ``feed(h, ctx)``; the engine may drop
                       rows of ``h`` between the two (only wanted rows go on after the last
                       mixer, as the reference does: src/models/qwen2/graph.rs:126-138)

The residual stream ``h`` is float32 [tokens, width]; ``x`` is a normed copy in the
activation dtype.  ``forward_add`` adds the part's output into ``h`` in float32.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..weights.spec import TensorSpec


@dataclass(frozen=True)
class CacheRequest:
    """Keys and values a mixer keeps per position.  ``window`` 0: every position is kept;
    otherwise only the last ``window`` positions are ever read."""

    n_kv_heads: int
    head_dim: int
    window: int = 0
    value_dim: int = 0       # width of a value vector if it differs from the keys' (0: head_dim)


@dataclass(frozen=True)
class StateRequest:
    """Per-sequence state of fixed size, zeroed when a slot is handed out."""

    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheView:
    """One cache entry as kernels see it."""

    k: torch.Tensor                 # [pages, n_kv_heads, 64, head_dim]
    v: torch.Tensor                 # [pages, n_kv_heads, 64, value_dim or head_dim]
    page_table: torch.Tensor        # int32 [batch rows, table_stride]
    table_stride: int
    ring: int                       # 0 = linear, else ring length in positions


@dataclass
class CallBinding:
    """What one entry of the run order gives its mixer: its cache entry (if the mixer asked
    for one), whether this call writes it, and its per-sequence state tensors
    ``[max_slots, *shape]`` by name."""

    cache: Optional[CacheView] = None
    writes_cache: bool = True
    entry: int = -1                 # which cache entry (calls that share keys name the same)
    has_readers: bool = False       # another call reads the entry this call writes
    state: Dict[str, torch.Tensor] = field(default_factory=dict)


@dataclass
class Pending:
    """A projection's output that has not been added into the residual stream yet: the
    float32 K splits ``partial`` [splits, rows, width] and an optional bias.  The true
    residual is ``h + bias + partial.sum(0)``.  The next norm adds it while it reads ``h``
    (``Norm.forward_settling``); anything else calls ``settle``."""

    partial: torch.Tensor
    bias: Optional[torch.Tensor] = None

    def settle(self, h: torch.Tensor) -> None:
        from ..kernels import api as K
        K.splitk_reduce(self.partial, self.bias, h, accumulate=True)


@dataclass
class Prepared:
    """What a product that completed the residual stream left for the norm that reads it next
    (``norm``): ``x`` = bfloat16(h * weight of that norm) and the sums of h^2 that give each
    row's 1/rms (``scale``, a ``kernels.api.RowScale``).  ``h`` itself is complete in memory, so
    anyone who cannot use this simply ignores it and norms ``h``."""

    x: torch.Tensor
    scale: Any
    norm: Any


def settle_pending(ctx: "StepContext", h: torch.Tensor) -> None:
    """Adds what a part left pending into ``h``."""
    pending = ctx.extras.pop("pending", None)
    if pending is not None:
        pending.settle(h)


@dataclass
class StepContext:
    """The batch of one step, as device tensors plus the few host numbers kernels need for
    their launch shape.  Row ``b`` of the batch is one sequence; tokens are packed row
    after row.  The engine may order the rows as it likes (logits go back in the caller's
    order): in a step where some rows bring one token and others more, the one-token rows come
    first and ``extras["single_rows"]`` says how many they are, so that a mixer can treat that
    stretch of tokens with its kernel for single tokens."""

    device: torch.device
    act_dtype: torch.dtype
    n_tokens: int
    n_rows: int
    token_ids: torch.Tensor         # int32 [n_tokens]
    positions: torch.Tensor         # int32 [n_tokens] absolute position of each token
    token_row: torch.Tensor         # int32 [n_tokens] batch row of each token
    cu_seqlens: torch.Tensor        # int32 [n_rows + 1]
    seq_end: torch.Tensor           # int32 [n_rows] sequence length after this step
    slots: torch.Tensor             # int32 [n_rows] slot of each row
    from_start: bool                # every row starts at position 0 (whole prompts)
    single_token: bool              # every row brings exactly one token
    max_row_tokens: int
    max_end: int                    # host: upper bound of seq_end (sizes key chunks)
    status: torch.Tensor            # int32 [1] error bits set by kernels
    host_slots: Sequence[int] = ()
    extras: Dict[str, Any] = field(default_factory=dict)
    # set by a block around a call of a mixer or feed-forward that says ``accepts_row_scale``:
    # the rows of ``x`` still lack their norm's 1/rms (a ``kernels.api.RowScale``), which the
    # part's first product applies
    input_scale: Any = None


class Part:
    """Common to all roles: the tensors wanted and how they are taken in.

    ``capturable``: the part only launches kernels on the current stream (no read of device
    memory on the host, no allocation the caching allocator cannot replay).  The engine
    replays decode steps as CUDA graphs only when every part of the model says so."""

    capturable = False

    def libraries(self, dtype: torch.dtype) -> List[str]:
        """Names of the kernel libraries this part launches from when the engine runs in
        ``dtype``; the engine compiles them side by side before the first step."""
        return []

    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        return []

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        """Takes its tensors (already on the device, in the precision they are held in)."""

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        """The tensors of ``tensor_specs`` by name, as held (views into packed storage where
        the part packed them at load)."""
        return {}


class ModelPart(Part):
    """A part of the model around the blocks (role ``"model"``), named by the plan: after the
    embedding (``ModelPlan.after_embedding``: learned positions added to the residual stream,
    for instance) or on the logits (``ModelPlan.on_logits``: a soft cap, for instance).  It
    changes its tensor in place, row by row: row ``t`` of ``h`` is token ``t`` of the step
    (``ctx.positions[t]``, ``ctx.token_row[t]``); the rows of the logits are the wanted places."""

    def forward_inplace(self, x: torch.Tensor, ctx: "StepContext") -> None:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x32: torch.Tensor, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def foldable(self) -> Optional[Tuple[torch.Tensor, float, int]]:
        """(weight float32 [size], eps, size) if this norm is y = x / rms(x) * weight, so that
        the product before it can prepare its input and the product after it apply 1/rms
        (``Prepared``); None for any other norm."""
        return None

    def forward_settling(self, h: torch.Tensor, pending: "Pending",
                         out_dtype: torch.dtype) -> torch.Tensor:
        """Adds ``pending`` into ``h`` and norms the result.  Norms that can do both in one
        kernel override this."""
        pending.settle(h)
        return self.forward(h, out_dtype)


class PositionEncoding(Part):
    def fused_rotary(self, device: torch.device) -> Optional[Tuple[torch.Tensor, int, int]]:
        """(inv_freq float64 [rotary_dim/2], rotary_dim, style) for the fused rotary kernel,
        or None if this encoding is not a rotation of pairs."""
        return None

    def apply(self, qkv32: torch.Tensor, ctx: StepContext, n_heads: int, n_kv_heads: int,
              head_dim: int) -> None:
        """Changes q and k inside ``qkv32`` [tokens, (n_heads + 2 n_kv) * head_dim] in place."""
        raise NotImplementedError


class Mixer(Part):
    # True: ``forward_add`` looks at ``ctx.input_scale`` and lets its first product apply it;
    # ``ctx.extras["prepare_for"]`` (a norm), if set, may be answered with a ``Prepared`` in
    # ``ctx.extras["prepared"]`` by the product that adds into the residual
    accepts_row_scale = False

    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_request(self) -> Sequence[StateRequest]:
        return ()

    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        raise NotImplementedError


class FeedForward(Part):
    accepts_row_scale = False      # as for ``Mixer``

    def forward_add(self, x: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def entry_norm(self) -> Optional[Norm]:
        """The norm that reads the residual stream first in ``mix``, if the block can take that
        norm's input prepared by the product before it (``Prepared``); else None."""
        return None

    def parts(self) -> Sequence[Part]:
        """Every part this block runs, whatever it calls them; the engine asks each whether it
        can be captured into a CUDA graph and which kernel libraries it needs."""
        raise NotImplementedError

    def mix(self, h: torch.Tensor, ctx: StepContext, binding: CallBinding) -> None:
        raise NotImplementedError

    def feed(self, h: torch.Tensor, ctx: StepContext) -> None:
        raise NotImplementedError
