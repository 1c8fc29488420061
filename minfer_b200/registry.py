"""One registry from an architecture's name to its model definition, and one from a
part's kind to its class.

The reference dispatches on the architecture string in one place
(src/models/mod.rs:74-87: ``"qwen2" => ...``, anything else prints
``Unsupported architecture`` and yields nothing).  Here the same decision is a table, so
that a new architecture or a new kind of part is one ``register_*`` call from any module,
including a test, with no change to the framework's files.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .config.base import ConfigError, ModelPlan, PartSpec

PART_ROLES = ("mixer", "feed_forward", "norm", "position", "block", "model")


@dataclass(frozen=True)
class ArchitectureDef:
    """``read_config(dict, where)`` returns the typed configuration; the configuration's
    ``plan()`` lowers it to a ``ModelPlan``."""

    name: str
    read_config: Callable[[Mapping[str, Any], str], Any]


_architectures: dict[str, ArchitectureDef] = {}
_parts: dict[str, dict[str, Callable[..., Any]]] = {role: {} for role in PART_ROLES}


class UnsupportedArchitecture(ConfigError):
    pass


def register_architecture(name: str, read_config: Callable[[Mapping[str, Any], str], Any],
                          replace: bool = False) -> None:
    if name in _architectures and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _architectures[name] = ArchitectureDef(name, read_config)


def known_architectures() -> list[str]:
    return sorted(_architectures)


def architecture_name(config: Mapping[str, Any], where: str = "config.json") -> str:
    archs = config.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: key 'architectures' must be a non-empty list of names")
    return archs[0]


def read_config(config: Mapping[str, Any], where: str = "config.json") -> Any:
    """The typed configuration of whatever architecture ``config`` names."""
    name = architecture_name(config, where)
    arch = _architectures.get(name)
    if arch is None:
        raise UnsupportedArchitecture(
            f"{where}: unsupported architecture '{name}' (known: {', '.join(known_architectures())})")
    return arch.read_config(config, where)


def plan_from_config(config: Mapping[str, Any], where: str = "config.json") -> ModelPlan:
    plan = read_config(config, where).plan()
    plan.validate()
    return plan


def register_part(role: str, kind: str, factory: Callable[..., Any], replace: bool = False) -> None:
    """``factory(**params)`` builds the part from its sizes and constants."""
    if role not in _parts:
        raise ValueError(f"unknown part role '{role}' (roles: {', '.join(PART_ROLES)})")
    if kind in _parts[role] and not replace:
        raise ValueError(f"{role} '{kind}' is already registered")
    _parts[role][kind] = factory


def known_parts(role: str) -> list[str]:
    return sorted(_parts[role])


def build_part(role: str, spec: PartSpec, **extra: Any) -> Any:
    table = _parts.get(role)
    if table is None:
        raise ValueError(f"unknown part role '{role}'")
    factory = table.get(spec.kind)
    if factory is None:
        raise ConfigError(
            f"no {role} of kind '{spec.kind}' is registered (known: {', '.join(known_parts(role))})")
    params = dict(spec.params)
    params.update(extra)
    return factory(**params)
