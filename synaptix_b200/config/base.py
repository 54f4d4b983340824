"""Typed model configuration: the base every architecture's config derives from.

A configuration is a frozen dataclass whose fields are read from the
architecture's own ``config.json`` keys.  No size and no constant that
``config.json`` gives is written anywhere else in the package: parts receive
their sizes and constants as constructor parameters, taken from here.

The reference keeps one serde struct per architecture with defaults and a
``validate`` method (crates/synaptix-models/llm/qwen3/src/config.rs:5-87) and
lowers it to a generic knob set (crates/synaptix-models/llm/common/src/config.rs:50-151).
Here the lowering is the architecture's ``build`` function, which turns the
typed config into parts (see ``synaptix_b200/models``).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar, Dict, Tuple


class ConfigError(ValueError):
    """A config.json that cannot be read, lacks a key, or names an unsupported option."""


_MISSING = object()


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all typed configurations.

    Subclasses declare ``architectures`` (the names in ``config.json``'s
    ``architectures`` list they answer to) and ``model_types`` (the
    ``model_type`` strings), implement ``from_dict`` and ``validate``, and
    ``to_dict`` so that a random-weights model folder can be written back.
    """

    architectures: ClassVar[Tuple[str, ...]] = ()
    model_types: ClassVar[Tuple[str, ...]] = ()

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError


def read_config_json(model_dir_or_file: str) -> Dict[str, Any]:
    """Read ``config.json`` (a folder holding one, or the file itself) into a dict."""
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    except json.JSONDecodeError as e:
        raise ConfigError(f"cannot parse {path}: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return d


def take(d: Dict[str, Any], key: str, typ, default=_MISSING, *, where: str = "config.json"):
    """Fetch ``key`` from ``d`` with a type check; a missing key without default is an error.

    ``typ`` is ``int``, ``float``, ``bool`` or ``str``.  JSON integers are
    accepted for floats; booleans are never accepted for numbers.
    """
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"{where}: required key '{key}' is missing")
        return default
    v = d[key]
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"{where}: '{key}' must be true or false, got {v!r}")
        return v
    if isinstance(v, bool):
        raise ConfigError(f"{where}: '{key}' must be {typ.__name__}, got {v!r}")
    if typ is int:
        if isinstance(v, float) and v.is_integer():
            v = int(v)
        if not isinstance(v, int):
            raise ConfigError(f"{where}: '{key}' must be an integer, got {v!r}")
        return v
    if typ is float:
        if not isinstance(v, (int, float)):
            raise ConfigError(f"{where}: '{key}' must be a number, got {v!r}")
        return float(v)
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"{where}: '{key}' must be a string, got {v!r}")
        return v
    raise TypeError(typ)
