"""Chooses the kernel of a bfloat16 x bfloat16 projection: the tcgen05 kernel whenever its
operands qualify (rows on 16-byte boundaries for TMA), else the FP32-pipe kernel."""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import api as K

_status: dict = {}
_current: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The device word the tensor-core kernels set bits in when a bounded wait runs out: the
    word of the engine whose step is running on ``device`` (``use_status_word``), else one
    word per device for products launched outside any engine."""
    key = str(device)
    word = _current.get(key)
    if word is not None:
        return word
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def use_status_word(word) -> None:
    """Products launched on the word's device from now on report into ``word`` (an engine
    calls this at the start of each of its steps); ``None`` has no effect."""
    if word is not None:
        _current[str(word.device)] = word


_USE_TENSOR_CORES = os.environ.get("MINFER_B200_NO_TCGEN05", "0") != "1"     # read once


def use_tensor_cores() -> bool:
    return _USE_TENSOR_CORES


def gemm_bf16(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
              out: torch.Tensor, accumulate: bool) -> None:
    if use_tensor_cores() and K.gemm_tc_supported(x, weight) and out.stride(1) == 1:
        K.gemm_tc(x, weight, bias, out, K.EPI_ACCUM if accumulate else K.EPI_STORE,
                  status_word(x.device))
    else:
        K.gemm_simt(x, weight, bias, out, accumulate)
