"""Random weights from a configuration and a seed.

The reference always maps weights from a file (src/models/qwen2/loader.rs:166-209); it
has no such mode.  Values depend only on (seed, tensor name), never on the order in
which tensors are made, so a folder written here and weights made in place agree.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Any, Mapping, Sequence

import torch

from .safetensors_io import save_file
from .spec import INT_TABLE, VECTOR, TensorSpec

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec: TensorSpec, seed: int, device: torch.device | str = "cpu") -> torch.Tensor:
    """float32 values ``mean + std * N(0,1)`` (integer tables: zeros)."""
    if spec.role == INT_TABLE:
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, spec.name))
    if spec.init.std == 0.0:
        return torch.full(spec.shape, spec.init.mean, dtype=torch.float32, device=device)
    t = torch.randn(spec.shape, generator=gen, dtype=torch.float32, device=device)
    return t.mul_(spec.init.std).add_(spec.init.mean)


def random_weights(specs: Sequence[TensorSpec], seed: int, store_dtype: torch.dtype,
                   device: torch.device | str = "cpu") -> dict[str, torch.Tensor]:
    """Every tensor of ``specs`` rounded once to ``store_dtype``."""
    out = {}
    for spec in specs:
        t = random_tensor(spec, seed, device)
        out[spec.name] = t if spec.role == INT_TABLE else t.to(store_dtype)
    return out


def write_model_folder(folder: str, config_json: Mapping[str, Any], specs: Sequence[TensorSpec],
                       seed: int, store_dtype: str | torch.dtype = "bfloat16") -> None:
    """Writes ``config.json`` and ``model.safetensors`` for a random model."""
    dtype = _STORE[store_dtype] if isinstance(store_dtype, str) else store_dtype
    os.makedirs(folder, exist_ok=True)
    tensors = random_weights(specs, seed, dtype, "cpu")
    save_file(tensors, os.path.join(folder, "model.safetensors"),
              metadata={"format": "pt", "seed": str(seed)})
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config_json), f, indent=2)
