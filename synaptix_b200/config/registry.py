"""One registry from an architecture's name to its configuration class and model builder.

The reference picks the architecture from ``config.json``'s ``model_type`` with
Qwen3 as the default arm (crates/synaptix/src/facade/arch.rs:62-83).  Here the
lookup is explicit: ``architectures[0]`` first, then ``model_type``; an unknown
name is an error that lists what is registered.

A builder is ``build(config, weights, runtime) -> Model`` (see
``synaptix_b200.models.qwen3.build`` for the one shipped).  Registering another
architecture needs no change to this file: call ``register_architecture`` from
the module that defines it.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, NamedTuple, Type

from .base import ConfigError, ModelConfig, read_config_json


class ArchitectureEntry(NamedTuple):
    name: str
    config_cls: Type[ModelConfig]
    build: Callable[..., Any]


_BY_ARCH: Dict[str, ArchitectureEntry] = {}
_BY_MODEL_TYPE: Dict[str, ArchitectureEntry] = {}


def register_architecture(config_cls: Type[ModelConfig], build: Callable[..., Any]) -> ArchitectureEntry:
    """Register ``config_cls`` under every name it declares; later registrations replace earlier ones."""
    if not config_cls.architectures:
        raise ValueError(f"{config_cls.__name__} declares no architecture names")
    entry = ArchitectureEntry(config_cls.architectures[0], config_cls, build)
    for a in config_cls.architectures:
        _BY_ARCH[a] = entry
    for t in config_cls.model_types:
        _BY_MODEL_TYPE[t] = entry
    return entry


def registered_architectures() -> List[str]:
    return sorted(_BY_ARCH)


def resolve_architecture(config_dict: Dict[str, Any]) -> ArchitectureEntry:
    """Find the registered architecture a parsed config.json asks for."""
    archs = config_dict.get("architectures")
    if isinstance(archs, list):
        for a in archs:
            if a in _BY_ARCH:
                return _BY_ARCH[a]
    mt = config_dict.get("model_type")
    if isinstance(mt, str) and mt in _BY_MODEL_TYPE:
        return _BY_MODEL_TYPE[mt]
    raise ConfigError(
        f"config.json names architectures={archs!r}, model_type={mt!r}; "
        f"registered architectures: {registered_architectures()}")


def load_config(model_dir_or_file: str) -> ModelConfig:
    """Read config.json and return the typed configuration of its architecture."""
    d = read_config_json(model_dir_or_file)
    return resolve_architecture(d).config_cls.from_dict(d)
