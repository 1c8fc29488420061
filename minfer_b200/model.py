"""A model: the plan's layers built from registered parts, with their weights on the device.

Counterpart of the reference's ``Qwen2Model`` (src/models/qwen2/mod.rs:13-76: hparams,
token embedding, output norm, output matrix, layers) and ``load_model``
(src/models/mod.rs:74-87), but nothing here names an architecture: the class of every
part comes from the plan.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any, Dict, List, Mapping, Optional, Sequence

import torch

from . import parts as _parts  # registers the shipped parts
from . import models as _models  # registers the shipped architectures
from .config.base import ModelPlan
from .parts.base import Block, Norm
from .parts.linear import Linear
from .registry import build_part, plan_from_config, read_config
from .weights.loader import held_dtype, load_weights
from .weights.random_init import random_tensor, write_model_folder
from .weights.spec import MATRIX, VECTOR, Init, TensorSpec

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def engine_dtype(dtype: Any) -> torch.dtype:
    try:
        return DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


class Model:
    def __init__(self, plan: ModelPlan, dtype: Any = "bfloat16", config: Any = None):
        plan.validate()
        self.plan = plan
        self.config = config
        self.dtype = engine_dtype(dtype)
        self.blocks: List[Block] = [build_part("block", layer.block, layer=layer)
                                    for layer in plan.layers]
        self.final_norm: Norm = build_part("norm", plan.final_norm)
        self.after_embedding = (build_part("model", plan.after_embedding)
                                if plan.after_embedding is not None else None)
        self.on_logits = build_part("model", plan.on_logits) if plan.on_logits is not None else None
        self.embedding: Optional[torch.Tensor] = None
        self.head: Optional[Linear] = None
        self.device: Optional[torch.device] = None

    # ---- what the checkpoint must hold --------------------------------------------------
    def tensor_specs(self) -> List[TensorSpec]:
        p = self.plan
        specs = [TensorSpec(p.embedding_name, (p.vocab_size, p.hidden_size), MATRIX, Init(0.0, 0.02))]
        for block in self.blocks:
            specs += block.tensor_specs()
        specs += self.final_norm.tensor_specs(p.final_norm_prefix)
        for part in self.model_parts():
            specs += part.tensor_specs(p.model_part_prefix)
        if p.head_name is not None:
            specs.append(TensorSpec(p.head_name, (p.vocab_size, p.hidden_size), MATRIX,
                                    Init(0.0, 0.02)))
        if p.head_bias_name is not None:
            specs.append(TensorSpec(p.head_bias_name, (p.vocab_size,), VECTOR, Init(0.0, 0.02)))
        names = [s.name for s in specs]
        if len(set(names)) != len(names):
            dup = sorted({n for n in names if names.count(n) > 1})
            raise ValueError(f"two parts ask for the same tensor: {', '.join(dup)}")
        return specs

    def model_parts(self) -> List[Any]:
        """The plan's parts around the blocks that this model has."""
        return [part for part in (self.after_embedding, self.on_logits) if part is not None]

    def ignorable_tensors(self) -> List[str]:
        """Names a checkpoint may hold without being used: a separate head beside tied
        embeddings (the reference uses the embedding table whenever there is no output
        matrix: src/models/qwen2/loader.rs:256-263)."""
        return ["lm_head.weight"] if self.plan.head_name is None else []

    # ---- taking weights in ----------------------------------------------------------------
    def bind(self, weights: Dict[str, torch.Tensor], device: torch.device | str) -> "Model":
        p = self.plan
        self.device = torch.device(device)
        self.embedding = weights[p.embedding_name]
        for block in self.blocks:
            block.load("", weights)
        self.final_norm.load(p.final_norm_prefix, weights)
        for part in self.model_parts():
            part.load(p.model_part_prefix, weights)
        head_w = self.embedding if p.head_name is None else weights[p.head_name]
        self.head = Linear(head_w, weights[p.head_bias_name] if p.head_bias_name is not None else None)
        return self

    @classmethod
    def from_folder(cls, folder: str, dtype: Any = "bfloat16",
                    device: torch.device | str = "cuda:0") -> "Model":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
        config = read_config(raw, path)
        model = cls(config.plan(), dtype, config)
        specs = model.tensor_specs()
        weights = load_weights(folder, specs, model.dtype, device, model.ignorable_tensors())
        return model.bind(weights, device)

    @classmethod
    def from_config(cls, config: Mapping[str, Any], seed: int = 0, dtype: Any = "bfloat16",
                    device: torch.device | str = "cuda:0", store_dtype: Any = None,
                    norm_std: float = 0.0, make_on: str = "cpu",
                    weight_std: Optional[float] = None) -> "Model":
        """Random weights without a folder.  Values are rounded once to ``store_dtype``
        (default: the engine dtype), as if read from a file of that precision.  They are
        drawn on ``make_on``: "cpu" gives the values ``write_random_model`` writes for the
        same seed; "device" draws on the target device (other values, much faster for
        billions of parameters)."""
        cfg = read_config(config, "config")
        model = cls(cfg.plan(), dtype, cfg)
        store = engine_dtype(store_dtype) if store_dtype is not None else model.dtype
        weights = {}
        for spec in with_norm_std(model.tensor_specs(), norm_std, weight_std):
            t = random_tensor(spec, seed, device if make_on == "device" else "cpu").to(device)
            if t.is_floating_point():
                t = t.to(store)
                t = t.to(held_dtype(spec, store, model.dtype))
            weights[spec.name] = t.contiguous()
        return model.bind(weights, device)

    # ---- the short way in: the same calls under the names a user of model libraries expects --
    @classmethod
    def from_pretrained(cls, folder: str, dtype: Any = "bfloat16",
                        device: torch.device | str = "cuda:0") -> "Model":
        """``from_folder`` under its usual name: config.json + model.safetensors -> model."""
        return cls.from_folder(folder, dtype, device)

    @classmethod
    def random(cls, config: Mapping[str, Any], seed: int = 0, dtype: Any = "bfloat16",
               device: torch.device | str = "cuda:0") -> "Model":
        """Seeded random weights for a configuration (``from_config`` with its defaults)."""
        return cls.from_config(config, seed, dtype, device)

    def new_session(self, max_seqs: int = 8, max_positions: int = 4096, cuda_graphs: bool = True):
        """An ``Engine`` over this model: a cache for ``max_seqs`` sequences of up to
        ``max_positions`` positions; ``acquire`` slots, ``step`` them, ``release`` them."""
        from .engine.step import Engine
        return Engine(self, max_tokens=max_seqs * max_positions, max_seqs=max_seqs,
                      cuda_graphs=cuda_graphs)

    def generate(self, prompts, max_new_tokens: int = 512, sampling=None, stop_token_ids=None,
                 max_batch: int = 8, max_positions: int = 4096):
        """Token ids in, ``GenerationResult``s out; builds a ``Generator`` for this call (keep
        a ``Generator`` yourself to reuse its cache and captured graphs)."""
        from .engine.generate import Generator
        gen = Generator(self, max_tokens=max_batch * max_positions, max_batch=max_batch)
        return gen.generate(prompts, max_new_tokens, sampling, stop_token_ids)

    def export_state_dict(self) -> Dict[str, torch.Tensor]:
        """The weights by their names in the checkpoint, as this model holds them (projections
        that were packed at load come back as views into the packed storage)."""
        p = self.plan
        out = {p.embedding_name: self.embedding}
        for block in self.blocks:
            out.update(block.export(""))
        out.update(self.final_norm.export(p.final_norm_prefix))
        for part in self.model_parts():
            out.update(part.export(p.model_part_prefix))
        if p.head_name is not None:
            out[p.head_name] = self.head.weight
        if p.head_bias_name is not None:
            out[p.head_bias_name] = self.head.bias
        return out

    # ---- sizes ----------------------------------------------------------------------------
    def parameter_bytes(self) -> int:
        """Bytes of all weights as held on the device, every storage counted once (a tied head
        is the embedding's storage; packed projections are one storage under several names).
        Asked of the parts through ``export_state_dict``, so a part that keeps its weights in
        any form is counted."""
        seen, total = set(), 0
        for t in self.export_state_dict().values():
            store = t.untyped_storage()
            if store.data_ptr() not in seen:
                seen.add(store.data_ptr())
                total += store.nbytes()
        return total


def with_norm_std(specs: Sequence[TensorSpec], norm_std: float,
                  weight_std: Optional[float] = None) -> List[TensorSpec]:
    """Norm weights drawn as 1 + N(0, norm_std) instead of exactly 1; with ``weight_std``
    every other tensor as N(0, weight_std) instead of its own default."""
    out = []
    for s in specs:
        if s.init.mean == 1.0:
            out.append(TensorSpec(s.name, s.shape, s.role, Init(1.0, norm_std)))
        elif weight_std is not None and s.init.std > 0.0:
            out.append(TensorSpec(s.name, s.shape, s.role, Init(s.init.mean, weight_std)))
        else:
            out.append(s)
    return out


def write_random_model(folder: str, config: Mapping[str, Any], seed: int,
                       store_dtype: str = "bfloat16", norm_std: float = 0.0,
                       weight_std: Optional[float] = None) -> None:
    """The random-weights mode: writes ``config.json`` and ``model.safetensors``."""
    cfg = read_config(config, "config")
    model = Model(cfg.plan(), "float32", cfg)
    out = dict(cfg.to_dict()) if hasattr(cfg, "to_dict") else dict(config)
    out["torch_dtype"] = store_dtype
    write_model_folder(folder, out, with_norm_std(model.tensor_specs(), norm_std, weight_std), seed,
                       store_dtype)
