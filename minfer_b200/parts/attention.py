"""Grouped-query attention as a mixer: fused q|k|v projection with bias, position encoding,
cache write, attention over the cache, output projection added into the residual stream.

Per layer the reference runs norm -> Wq/Wk/Wv (+bias) -> rotary on q and k -> KV store ->
attention -> Wo -> residual (src/models/qwen2/graph.rs:63-137); its Metal path packs
wq|wk|wv into one matrix followed by one bias+rotary+store pass
(src/models/qwen2/graph.rs:69-98, src/models/qwen2/loader.rs:290-331).  Here the packed
projection is the only path: one product, then one kernel that rotates and writes the
cache, then attention, then Wo with the residual add in its epilogue.

Whole prompts (every row of the step starts at position 0) attend over the step's own keys
and values; any other step (one token a row, a prompt's later portion, a mix of both)
attends over the cache, which by then holds the step's keys too: every token is a query at
its own absolute position.  All sizes are parameters.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..config.base import PartSpec
from ..kernels import api as K
from ..weights.spec import MATRIX, VECTOR, Init, TensorSpec
from .base import CacheRequest, CallBinding, Mixer, StepContext, settle_pending
from .linear import Linear

DECODE_CHUNK = 256     # keys per block when attending over the cache
_DECODE_CTAS = os.environ.get("MINFER_B200_DECODE_CTAS")
_decode_ctas_of: Dict[int, int] = {}


def decode_ctas(device: Optional[torch.device] = None) -> int:
    """CTAs the decode kernel wants in flight: two on each SM of the device."""
    if _DECODE_CTAS:
        return int(_DECODE_CTAS)
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _decode_ctas_of:
        _decode_ctas_of[index] = 2 * torch.cuda.get_device_properties(index).multi_processor_count
    return _decode_ctas_of[index]


FORCE_GENERIC_ATTENTION = os.environ.get("MINFER_B200_GENERIC_ATTENTION", "0") == "1"
# a step that is neither whole prompts nor one token a row runs the tcgen05 kernel over the
# cache's pages from this many tokens on; below, every token is a row of the decode kernel
# (a query tile of 128 rows for a handful of tokens wastes the tensor cores' time, and few
# rows give that kernel few CTAs).  Measured at 2,048 cached positions, 4 layers of the 7B
# shape: 8 rows x 16 tokens 1.17 ms against 1.06 with the decode kernel, 8 x 32 1.46 against
# 1.76, 7 rows of one token beside one of 512 2.17 against 2.98.
PAGED_PROMPT_MIN_TOKENS = int(os.environ.get("MINFER_B200_PAGED_PROMPT_MIN_TOKENS", "160"))
# "tcgen05" (tensor memory, the default) or "mma" (the mma.sync twin) for whole prompts in bfloat16
PROMPT_ATTENTION = os.environ.get("MINFER_B200_PROMPT_ATTENTION", "tcgen05")


def decode_chunks(items: int, max_end: int, tensor_cores: bool = True,
                  ctas: Optional[int] = None) -> tuple:
    """How attention over the cache cuts the keys: (keys per chunk, chunks).  A chunk is a
    CTA's work and a multiple of 256 keys.  The tensor-core kernel is fastest when the CTAs of
    all ``items`` (rows x key/value heads) fill the GPU about once, two to an SM: with few
    items or long contexts a CTA then walks several blocks of 256 keys (8 sequences at 8,192
    positions: 36.7 us with 4 blocks a CTA against 46.0 with one; at 32,000: 108 against
    157 us), and fewer chunks are left to merge."""
    blocks = max(1, -(-max_end // DECODE_CHUNK))
    if not tensor_cores:
        return DECODE_CHUNK, blocks
    if ctas is None:
        ctas = decode_ctas()
    if items * blocks <= ctas * 3 // 2:
        return DECODE_CHUNK, blocks                    # one block a CTA: up to three CTAs on an SM
    n_chunks = max(1, min(blocks, ctas // max(items, 1)))
    per = -(-blocks // n_chunks)
    return per * DECODE_CHUNK, -(-blocks // per)


class Attention(Mixer):
    capturable = True      # launches kernels only; safe inside a CUDA graph capture

    def libraries(self, dtype: torch.dtype) -> List[str]:
        libs = ["ops", "attention"]
        if dtype == torch.bfloat16:
            libs += ["gemm_tc", "attention_prefill_tc"]
        else:
            libs.append("gemm_simt")
        return libs

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, window: int = 0, qkv_bias: bool = True, out_bias: bool = False,
                 position: Optional[PartSpec] = None, init_std: float = 0.02):
        from ..registry import build_part
        if n_heads % n_kv_heads != 0:
            raise ValueError(f"{n_heads} heads do not divide into {n_kv_heads} key/value heads")
        if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
            raise ValueError(
                f"head size {head_dim} is not supported: the attention kernels take multiples "
                f"of 16 from 16 to 256")
        self.hidden_size = int(hidden_size)
        self.n_heads = int(n_heads)
        self.n_kv_heads = int(n_kv_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = int(window)
        self.qkv_bias = bool(qkv_bias)
        self.out_bias = bool(out_bias)
        self.init_std = float(init_std)
        self.position = build_part("position", position) if position is not None else None
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None

    # ---- weights ----------------------------------------------------------------------
    def tensor_specs(self, prefix: str) -> List[TensorSpec]:
        p = f"{prefix}self_attn."
        nq, nkv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        init = Init(0.0, self.init_std)
        specs = [TensorSpec(f"{p}q_proj.weight", (nq, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}k_proj.weight", (nkv, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}v_proj.weight", (nkv, self.hidden_size), MATRIX, init),
                 TensorSpec(f"{p}o_proj.weight", (self.hidden_size, nq), MATRIX, init)]
        if self.qkv_bias:
            specs += [TensorSpec(f"{p}q_proj.bias", (nq,), VECTOR, init),
                      TensorSpec(f"{p}k_proj.bias", (nkv,), VECTOR, init),
                      TensorSpec(f"{p}v_proj.bias", (nkv,), VECTOR, init)]
        if self.out_bias:
            specs.append(TensorSpec(f"{p}o_proj.bias", (self.hidden_size,), VECTOR, init))
        if self.position is not None:
            specs += self.position.tensor_specs(p)
        return specs

    def load(self, prefix: str, weights: Dict[str, torch.Tensor]) -> None:
        p = f"{prefix}self_attn."
        parts = [weights[f"{p}{n}_proj.weight"] for n in "qkv"]
        if len({t.dtype for t in parts}) != 1:
            parts = [t.to(torch.float32) for t in parts]
        w = torch.cat(parts, dim=0).contiguous()
        b = None
        if self.qkv_bias:
            b = torch.cat([weights[f"{p}{n}_proj.bias"] for n in "qkv"]).contiguous()
        self.qkv = Linear(w, b)
        self.out = Linear(weights[f"{p}o_proj.weight"],
                          weights[f"{p}o_proj.bias"] if self.out_bias else None)
        # the projection of q|k|v can apply a norm's 1/rms itself (bfloat16 on tensor cores)
        self.accepts_row_scale = self.qkv.takes_row_scale()
        if self.position is not None:
            self.position.load(p, weights)

    def export(self, prefix: str) -> Dict[str, torch.Tensor]:
        p = f"{prefix}self_attn."
        nq, nkv = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim
        out = {}
        for name, lo, hi in (("q", 0, nq), ("k", nq, nq + nkv), ("v", nq + nkv, nq + 2 * nkv)):
            out[f"{p}{name}_proj.weight"] = self.qkv.weight[lo:hi]
            if self.qkv_bias:
                out[f"{p}{name}_proj.bias"] = self.qkv.bias[lo:hi]
        out[f"{p}o_proj.weight"] = self.out.weight
        if self.out_bias:
            out[f"{p}o_proj.bias"] = self.out.bias
        if self.position is not None:
            out.update(self.position.export(p))
        return out

    # ---- what it keeps per sequence -----------------------------------------------------
    def cache_request(self) -> Optional[CacheRequest]:
        return CacheRequest(self.n_kv_heads, self.head_dim, self.window)

    # ---- the step -----------------------------------------------------------------------
    def forward_add(self, x: torch.Tensor, ctx: StepContext, binding: CallBinding,
                    residual: torch.Tensor) -> None:
        n = x.shape[0]
        nh, nk, hd = self.n_heads, self.n_kv_heads, self.head_dim
        dev, act = x.device, ctx.act_dtype
        inv_freq, rotary_dim, style = None, 0, 0
        fused = self.position.fused_rotary(dev) if self.position is not None else (None, 0, 0)
        rs = ctx.input_scale                       # the norm's 1/rms, if this product is to apply it
        # the K splits of a small projection are added by the rotary kernel itself
        split = self.qkv.partial_sums(x, row_scale=rs) if fused is not None else None
        if split is not None:
            qkv, n_partials, qkv_bias = split.partial, split.partial.shape[0], split.bias
        else:
            qkv, n_partials, qkv_bias = self.qkv.forward(x, torch.float32, row_scale=rs), 0, None
        if fused is None:
            self.position.apply(qkv, ctx, nh, nk, hd)
        else:
            inv_freq, rotary_dim, style = fused

        cache = binding.cache
        if cache is None:
            raise K.KernelError("the attention mixer was given no cache entry")
        q = torch.empty((n, nh, hd), dtype=act, device=dev)
        write = binding.writes_cache
        own_kv = ctx.from_start
        k_step = v_step = None
        if own_kv and write:
            k_step = torch.empty((n, nk, hd), dtype=act, device=dev)
            v_step = torch.empty((n, nk, hd), dtype=act, device=dev)
            if binding.has_readers:
                ctx.extras[("step_kv", binding.entry)] = (k_step, v_step)
        elif own_kv:
            # whole prompts of a call that reads another call's entry: that call's keys
            k_step, v_step = ctx.extras[("step_kv", binding.entry)]
        if cache.k.dtype != act:
            raise K.KernelError("the cache and the activations must share one dtype")
        K.rope_kvstore(qkv, ctx.positions, ctx.token_row, ctx.seq_end, inv_freq, q,
                       k_step if write else None, v_step if write else None,
                       cache.k if write else None, cache.v if write else None,
                       cache.page_table if write else None, cache.table_stride, cache.ring,
                       nh, nk, hd, rotary_dim, style, ctx.status, n_partials=n_partials,
                       bias=qkv_bias)

        o = torch.empty((n, nh * hd), dtype=act, device=dev)
        if own_kv:
            if K.attention_prefill_supported(q, nh, nk, hd) and not FORCE_GENERIC_ATTENTION:
                if PROMPT_ATTENTION == "mma":
                    K.attention_prefill(q, k_step, v_step, ctx.cu_seqlens, o, ctx.n_rows,
                                        ctx.max_row_tokens, nh, nk, hd, self.window, self.scale)
                else:
                    K.attention_prefill_tc(q, k_step, v_step, ctx.cu_seqlens, o, ctx.n_rows,
                                           ctx.max_row_tokens, nh, nk, hd, self.window, self.scale,
                                           ctx.status)
            else:
                K.attention_packed(q, k_step, v_step, ctx.token_row, ctx.positions,
                                   ctx.cu_seqlens, o, nh, nk, hd, self.window, self.scale)
        else:
            # keys and values come from the cache, the step's own among them: each token is a
            # query at its position
            if cache.ring and ctx.max_row_tokens > cache.ring - self.window + 1:
                raise K.KernelError(
                    f"a sequence brings {ctx.max_row_tokens} tokens, but a ring of {cache.ring} "
                    f"positions with a window of {self.window} takes "
                    f"{cache.ring - self.window + 1} a step (the engine runs longer rows in portions)")
            n_one = int(ctx.extras.get("single_rows", 0))      # rows of one token, first in the batch
            if (not ctx.single_token and PROMPT_ATTENTION != "mma" and not FORCE_GENERIC_ATTENTION
                    and K.attention_prefill_supported(q, nh, nk, hd)
                    and ctx.n_tokens - n_one >= PAGED_PROMPT_MIN_TOKENS):
                # rows of several tokens: query tiles of the step's rows over the cache's pages
                stride = cache.table_stride
                K.attention_prefill_tc_paged(q, cache.k, cache.v, ctx.cu_seqlens[n_one:],
                                             ctx.seq_end[n_one:], cache.page_table[n_one * stride:],
                                             stride, cache.ring, o, ctx.n_rows - n_one,
                                             ctx.max_row_tokens, nh, nk, hd, self.window, self.scale,
                                             ctx.status)
                if n_one:
                    # the rows of one token beside them: the decode kernel, a row per token (each
                    # is its sequence's only new token, so its older keys were there before the step)
                    self._over_cache(q[:n_one], o[:n_one], ctx.token_row[:n_one], ctx.positions[:n_one],
                                     cache, ctx, final=True)
                self._project_out(o, ctx, residual)
                return
            self._over_cache(q, o, ctx.token_row, ctx.positions, cache, ctx, final=ctx.single_token)
        self._project_out(o, ctx, residual)

    def _over_cache(self, q: torch.Tensor, o: torch.Tensor, token_row: torch.Tensor,
                    positions: torch.Tensor, cache, ctx: StepContext, final: bool) -> None:
        """Every token of ``q`` a query at its position over the paged cache (key chunks and
        their merge).  ``final``: each is its sequence's only new token in this step."""
        n, act = q.shape[0], q.dtype
        nh, nk, hd = self.n_heads, self.n_kv_heads, self.head_dim
        chunk, n_chunks = decode_chunks(n * nk, ctx.max_end, tensor_cores=(
            act == torch.bfloat16 and hd in (64, 128) and nh // nk <= 16
            and not FORCE_GENERIC_ATTENTION))
        partial = None
        if n_chunks > 1 or act == torch.bfloat16:
            partial = torch.empty((n * nh * n_chunks * (hd + 2),), dtype=torch.float32,
                                  device=q.device)
        K.attention_paged(q, cache.k, cache.v, token_row, positions, cache.page_table,
                          cache.table_stride, cache.ring, o, partial, nh, nk, hd, self.window,
                          chunk, n_chunks, self.scale, force_generic=FORCE_GENERIC_ATTENTION,
                          status=ctx.status, old_keys_final=final)

    def _project_out(self, o: torch.Tensor, ctx: StepContext, residual: torch.Tensor) -> None:
        target = ctx.extras.pop("prepare_for", None)
        if target is not None:
            # the product completes the residual and prepares the next norm's input
            settle_pending(ctx, residual)
            prepared = self.out.accumulate_prepared(o, residual, target)
            if prepared is not None:
                ctx.extras["prepared"] = prepared
                return
        pending = self.out.partial_sums(o)
        if pending is None:
            self.out.forward(o, torch.float32, out=residual, accumulate=True)
        else:
            settle_pending(ctx, residual)          # never two at once
            ctx.extras["pending"] = pending
