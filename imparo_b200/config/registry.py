"""One registry from an architecture's name to its model.

The reference matches the file's architecture string to a plan builder and a
workflow, and adding a model is one module plus one row
(imparo-model/src/lib.rs:2929-2970 build_plan/load; lfm2/mod.rs:16-33).  Here a row
holds the typed config class and the function that turns a config into a
ModelSpec; everything below the spec is shared.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Tuple

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str                                   # e.g. "Lfm2ForCausalLM"
    model_types: Tuple[str, ...]                # accepted config.json "model_type" values
    parse_config: Callable[[dict], object]      # config.json dict -> typed config
    model_spec: Callable[[object], object]      # typed config -> parts.spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{arch.name}' is already registered")
    _ARCHITECTURES[arch.name] = arch


def known_architectures() -> Tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_ARCHITECTURES))


def _ensure_builtin() -> None:
    # The built-in architectures register themselves on import.
    from .. import models  # noqa: F401


def resolve_architecture(values: dict) -> Architecture:
    """Pick the architecture a config.json names: "architectures"[0], else "model_type".
    Unknown name -> error listing the known ones (PlanError::UnknownArchitecture)."""
    _ensure_builtin()
    names = values.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = values.get("model_type")
    if mt is not None:
        for arch in _ARCHITECTURES.values():
            if mt in arch.model_types:
                return arch
    asked = ", ".join(map(str, names)) or (str(mt) if mt is not None else "(none given)")
    raise ConfigError(f"config.json names architecture {asked}; known: {', '.join(sorted(_ARCHITECTURES))}")


def load_config(folder_or_dict):
    """-> (Architecture, typed config)."""
    values = folder_or_dict if isinstance(folder_or_dict, dict) else read_config_json(folder_or_dict)
    arch = resolve_architecture(values)
    return arch, arch.parse_config(values)
