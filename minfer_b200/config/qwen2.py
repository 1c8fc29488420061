"""Typed configuration of the Qwen2 dense decoder, read from its own config.json keys.

Counterpart of the reference's ``HParams`` (src/models/qwen2/loader.rs:11-39) and
``hparams_from_gguf`` (src/models/qwen2/loader.rs:97-147): required sizes fail when
missing, optional ones default as there (KV heads = heads :117-119, context 32768
:130-132, eps 1e-6 :133-135, rope base 10000 :136-138, frequency scale 1.0 :139-141),
the head size is hidden_size / heads (:32-34) and the attention scale 1/sqrt(head size)
(:36-38).  The sliding-window keys have no counterpart in the reference; their meaning
is fixed here: layer ``l`` is windowed iff ``use_sliding_window`` and
``l >= max_window_layers``, and a windowed query at position p sees keys j with
``0 <= p - j < sliding_window``.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional

from .base import (ConfigError, ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule)

ARCHITECTURE = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    rope_frequency_scale: float = 1.0
    max_position_embeddings: int = 32768
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_ids: tuple[int, ...] = ()
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    # ---- derived -------------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def attention_scale(self) -> float:
        return 1.0 / math.sqrt(self.head_dim)

    def layer_window(self, layer: int) -> int:
        """Window of a layer in positions, 0 for a layer that sees every earlier key."""
        if self.use_sliding_window and layer >= int(self.max_window_layers):
            return int(self.sliding_window)
        return 0

    # ---- reading --------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = ConfigReader(data, where)
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        kv_heads = r.integer("num_key_value_heads", default=heads, minimum=1)
        cfg = cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=hidden,
            num_hidden_layers=r.integer("num_hidden_layers", minimum=1),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            rms_norm_eps=r.number("rms_norm_eps", default=1e-6, positive=True),
            rope_theta=r.number("rope_theta", default=10000.0, positive=True),
            rope_frequency_scale=1.0,
            max_position_embeddings=r.integer("max_position_embeddings", default=32768, minimum=1),
            tie_word_embeddings=r.boolean("tie_word_embeddings", default=False),
            use_sliding_window=r.boolean("use_sliding_window", default=False),
            sliding_window=r.optional_integer("sliding_window", minimum=1),
            max_window_layers=r.optional_integer("max_window_layers", minimum=0),
            eos_token_ids=tuple(r.int_list("eos_token_id", default=[])),
            torch_dtype=r.string("torch_dtype", default=r.string("dtype", default="bfloat16")),
            extra={k: v for k, v in data.items()},
        )
        cfg._check(r, data)
        return cfg

    def _check(self, r: ConfigReader, data: Mapping[str, Any]) -> None:
        w = r.where
        if self.hidden_size % self.num_attention_heads != 0:
            raise ConfigError(
                f"{w}: hidden_size {self.hidden_size} is not a multiple of num_attention_heads "
                f"{self.num_attention_heads}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"{w}: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if "head_dim" in data and data["head_dim"] is not None and data["head_dim"] != self.head_dim:
            raise ConfigError(
                f"{w}: head_dim {data['head_dim']} differs from hidden_size / num_attention_heads "
                f"= {self.head_dim}; this architecture has no separate head size")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"{w}: the head size {self.head_dim} must be even for rotary pairs")
        act = data.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{w}: hidden_act must be 'silu' for this architecture, got {act!r}")
        if data.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"{w}: rope_scaling is not supported for this architecture")
        if self.use_sliding_window:
            if self.sliding_window is None:
                raise ConfigError(f"{w}: use_sliding_window is true but 'sliding_window' is missing")
            if self.max_window_layers is None:
                raise ConfigError(
                    f"{w}: use_sliding_window is true but 'max_window_layers' is missing")
        for t in self.eos_token_ids:
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"{w}: eos_token_id {t} is outside the vocabulary")

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen2Config":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), where=path)

    # ---- writing (random-weights mode writes a folder) ------------------------------
    def to_dict(self) -> dict:
        d = {
            "architectures": [ARCHITECTURE],
            "model_type": "qwen2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "intermediate_size": self.intermediate_size,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": self.use_sliding_window,
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["sliding_window"] = self.sliding_window
        if self.max_window_layers is not None:
            d["max_window_layers"] = self.max_window_layers
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        return d

    # ---- lowering to parts ----------------------------------------------------------
    def plan(self) -> ModelPlan:
        """Qwen2 as parts: per layer RMSNorm -> GQA attention with q/k/v bias and NeoX
        rotary -> residual -> RMSNorm -> SwiGLU -> residual
        (src/models/qwen2/graph.rs:59-177), final RMSNorm and head (:180-182)."""
        norm = PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        layers = []
        for l in range(self.num_hidden_layers):
            position = PartSpec("rotary", {
                "head_dim": self.head_dim,
                "rotary_dim": self.head_dim,
                "theta": self.rope_theta,
                "frequency_scale": self.rope_frequency_scale,
                "style": "neox",
            })
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size,
                "n_heads": self.num_attention_heads,
                "n_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": self.attention_scale,
                "window": self.layer_window(l),
                "qkv_bias": True,
                "out_bias": False,
                "position": position,
            })
            ffn = PartSpec("gated_mlp", {
                "hidden_size": self.hidden_size,
                "intermediate_size": self.intermediate_size,
                "activation": "silu",
            })
            layers.append(LayerSpec(
                prefix=f"model.layers.{l}.",
                block=PartSpec("pre_norm", {}),
                mixer=mixer,
                mixer_norm=norm.with_params(name="input_layernorm"),
                feed_forward=ffn,
                feed_forward_norm=norm.with_params(name="post_attention_layernorm"),
            ))
        plan = ModelPlan(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            embedding_name="model.embed_tokens.weight",
            head_name=None if self.tie_word_embeddings else "lm_head.weight",
            final_norm=norm.with_params(name="norm"),
            final_norm_prefix="model.",
            layers=layers,
            schedule=default_schedule(self.num_hidden_layers),
            max_positions=self.max_position_embeddings,
            stop_token_ids=tuple(self.eos_token_ids),
        )
        plan.validate()
        return plan
