"""Weights from a model folder by tensor name.

The reference looks every tensor up by name (src/models/qwen2/loader.rs:234-251; the
names are listed in src/models/qwen2/mod.rs:97-115), falls back to the embedding table
when there is no output matrix (loader.rs:256-263) and discovers a missing layer tensor
only as a panic at graph build (src/models/qwen2/graph.rs:100).  Here every expected
tensor is checked before anything is uploaded and ONE error lists all that is wrong:
missing names, unexpected names and wrong shapes.

Precision: matrices are kept in bfloat16 when the engine runs in bfloat16, except that
a tensor the file stores in 32-bit stays in 32-bit; in the float32 engine everything is
float32.  Norm weights and biases are always held in float32 (exact for bfloat16 files).
Integer tables become int32.
"""
from __future__ import annotations

import sys

from typing import Iterable, Mapping, Sequence

import torch

from .safetensors_io import Checkpoint, SafetensorsError
from .spec import INT_TABLE, MATRIX, VECTOR, TensorSpec

_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected``, ``wrong_shape``
    and ``wrong_type`` hold the offending names; the message lists all of them."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[tuple], wrong_type: Sequence[tuple]):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = [f"{where}: the checkpoint does not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(
                f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong types ({len(self.wrong_type)}): " + ", ".join(
                f"{n} is {got}, expected {want}" for n, got, want in self.wrong_type))
        super().__init__("\n".join(lines))


def held_dtype(spec: TensorSpec, stored: torch.dtype, engine_dtype: torch.dtype) -> torch.dtype:
    """The precision a tensor is kept in on the device."""
    if spec.role == INT_TABLE:
        return torch.int32
    if spec.role == VECTOR:
        return torch.float32
    if engine_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32          # a tensor stored in 32-bit stays so
    return torch.bfloat16


def check_against(specs: Sequence[TensorSpec], found: Mapping[str, tuple], where: str,
                  ignorable: Iterable[str] = ()) -> None:
    """``found`` maps a name to (shape, dtype).  Raises one ``WeightError`` for everything."""
    want = {s.name: s for s in specs}
    ignore = set(ignorable)
    missing = [n for n in want if n not in found]
    unexpected = [n for n in found if n not in want and n not in ignore]
    wrong_shape, wrong_type = [], []
    for name, spec in want.items():
        if name not in found:
            continue
        shape, dtype = found[name]
        if tuple(shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(shape), tuple(spec.shape)))
        if spec.role == INT_TABLE:
            if dtype not in _INTS:
                wrong_type.append((name, str(dtype), "an integer type"))
        elif dtype not in _FLOATS:
            wrong_type.append((name, str(dtype), "a floating-point type"))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(where, sorted(missing), sorted(unexpected), wrong_shape, wrong_type)


def load_weights(folder: str, specs: Sequence[TensorSpec], engine_dtype: torch.dtype,
                 device: torch.device | str, ignorable: Iterable[str] = ()) -> dict[str, torch.Tensor]:
    """Reads every tensor ``specs`` names, checks all of them first, then uploads."""
    try:
        ck = Checkpoint(folder)
    except SafetensorsError:
        raise
    try:
        found = {n: (ck.entry(n).shape, ck.entry(n).dtype) for n in ck.names()}
        check_against(specs, found, folder, ignorable)
        out: dict[str, torch.Tensor] = {}
        wide = []
        for spec in specs:
            t = ck.tensor(spec.name)
            held = held_dtype(spec, t.dtype, engine_dtype)
            if (engine_dtype == torch.bfloat16 and held == torch.float32
                    and spec.role not in (VECTOR, INT_TABLE)):
                wide.append(spec.name)
            out[spec.name] = t.to(held).to(device).contiguous()
        if wide:
            # kept as stored, as the rule says, but the user should know what it costs
            print(f"[minfer_b200] {len(wide)} matrices of {folder} are stored in 32-bit and stay "
                  f"float32 in the bfloat16 engine: their products run on the FP32 pipe (about "
                  f"40 times slower) and take twice the memory; store them in bfloat16 to use "
                  f"the tensor cores ({', '.join(wide[:3])}{', ...' if len(wide) > 3 else ''})",
                  file=sys.stderr, flush=True)
        return out
    finally:
        ck.close()
