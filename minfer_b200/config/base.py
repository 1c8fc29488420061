"""Architecture-independent description of a model: which parts each layer is made of,
with which sizes and constants, and in which order the layers run.

An architecture's own configuration class (for instance ``Qwen2Config``) reads its
``config.json`` keys into typed fields and then *lowers* itself into a ``ModelPlan``:
pure data that the part registry turns into runnable layers.  Nothing below the plan
knows which model it belongs to.

The reference carries the same information as per-node metadata of its compute graph
(eps, rope base/scale, head counts and the attention scale travel with each node:
src/graph/ops.rs:148-167) and fixes the layer order by build order
(src/models/qwen2/graph.rs:59-177); here both are explicit data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Sequence


class ConfigError(ValueError):
    """A configuration key is missing, has the wrong type, or breaks a constraint."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered kind and its parameters (sizes, constants)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def with_params(self, **extra: Any) -> "PartSpec":
        merged = dict(self.params)
        merged.update(extra)
        return PartSpec(self.kind, merged)


@dataclass(frozen=True)
class LayerSpec:
    """The parts one layer is put together from.

    ``prefix`` is the tensor-name prefix of the layer in the checkpoint
    (for instance ``model.layers.3.``).
    """

    prefix: str
    block: PartSpec
    mixer: PartSpec
    mixer_norm: PartSpec
    feed_forward: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer``      index into ``ModelPlan.layers`` (a layer may be named more than once).
    ``cache``      index of the cache entry this call uses; by default every call has an
                   entry of its own.  Two calls that name the same entry share keys and
                   values: the first of them in run order writes, the others only read
                   (``writes_cache`` False).
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelPlan:
    """Everything the engine needs to build a model, as data."""

    architecture: str
    vocab_size: int
    hidden_size: int
    embedding_name: str
    head_name: Optional[str]          # None: the head shares the embedding table
    final_norm: PartSpec
    final_norm_prefix: str
    layers: Sequence[LayerSpec]
    schedule: Sequence[LayerCall]
    max_positions: int
    stop_token_ids: Sequence[int] = ()
    # what some architectures do around the blocks (this one does neither): a factor on the
    # embedding rows as they enter the residual stream, a bias added to the logits
    embedding_scale: float = 1.0
    head_bias_name: Optional[str] = None
    # optional parts of role "model" (``ModelPart``) run on the residual stream right after the
    # embedding and on the logits right after the head; their tensors take this prefix
    after_embedding: Optional[PartSpec] = None
    on_logits: Optional[PartSpec] = None
    model_part_prefix: str = ""

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ConfigError("vocab_size and hidden_size must be positive")
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        if not self.schedule:
            raise ConfigError("the run order (schedule) is empty")
        writers: dict[int, int] = {}
        for i, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.layers):
                raise ConfigError(
                    f"schedule[{i}] names layer {call.layer}, but there are {len(self.layers)} layers")
            if call.cache < 0:
                raise ConfigError(f"schedule[{i}] has a negative cache entry {call.cache}")
            if call.writes_cache:
                if call.cache in writers:
                    raise ConfigError(
                        f"schedule[{i}] and schedule[{writers[call.cache]}] both write cache entry "
                        f"{call.cache}; only one call may write an entry")
                writers[call.cache] = i
        for i, call in enumerate(self.schedule):
            if not call.writes_cache:
                if call.cache not in writers:
                    raise ConfigError(
                        f"schedule[{i}] reads cache entry {call.cache}, which no call writes")
                if writers[call.cache] > i:
                    raise ConfigError(
                        f"schedule[{i}] reads cache entry {call.cache} before schedule"
                        f"[{writers[call.cache]}] has written it")


def default_schedule(n_layers: int) -> list[LayerCall]:
    """Every layer once, in order, each with a cache entry of its own."""
    return [LayerCall(layer=i, cache=i) for i in range(n_layers)]


# ---------------------------------------------------------------------------------------
# typed access to a config.json dictionary
# ---------------------------------------------------------------------------------------

_MISSING = object()


class ConfigReader:
    """Reads typed values out of a ``config.json`` dictionary with errors that name the key."""

    def __init__(self, data: Mapping[str, Any], where: str = "config.json"):
        if not isinstance(data, Mapping):
            raise ConfigError(f"{where}: expected a JSON object at the top level")
        self.data = data
        self.where = where

    def _get(self, key: str, default: Any) -> Any:
        value = self.data.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return value

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> int:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                value = int(value)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {value!r}")
        if minimum is not None and value < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {value}")
        return value

    def optional_integer(self, key: str, minimum: Optional[int] = None) -> Optional[int]:
        if self.data.get(key) is None:
            return None
        return self.integer(key, minimum=minimum)

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> float:
        value = self._get(key, default)
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {value!r}")
        value = float(value)
        if positive and not value > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {value}")
        return value

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        value = self._get(key, default)
        if not isinstance(value, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {value!r}")
        return value

    def string(self, key: str, default: Any = _MISSING) -> str:
        value = self._get(key, default)
        if not isinstance(value, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {value!r}")
        return value

    def int_list(self, key: str, default: Any = _MISSING) -> list[int]:
        """An integer or a list of integers (``eos_token_id`` comes in both forms)."""
        value = self._get(key, default)
        if isinstance(value, int) and not isinstance(value, bool):
            return [value]
        if isinstance(value, (list, tuple)) and all(
                isinstance(v, int) and not isinstance(v, bool) for v in value):
            return list(value)
        raise ConfigError(
            f"{self.where}: key '{key}' must be an integer or a list of integers, got {value!r}")
