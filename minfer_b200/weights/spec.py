"""What a model expects to find in a checkpoint: one ``TensorSpec`` per tensor."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

MATRIX = "matrix"        # operand of a matrix product or a lookup table of rows
VECTOR = "vector"        # norm weight, bias: always held in 32-bit
INT_TABLE = "int_table"  # integer table: held as int32


@dataclass(frozen=True)
class Init:
    """How the random-weights mode fills a tensor: ``mean + std * N(0, 1)``."""

    mean: float = 0.0
    std: float = 0.0


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    role: str = MATRIX
    init: Init = Init(0.0, 0.02)
