"""One registry from an architecture's name to its configuration class and model recipe.

The reference selects its model with an enum and an if/else on
``architectures[0]`` (src/model/model.cpp:14-20, 66-77).  Here the same string
is a key into a table, so that another architecture is one ``register`` call:
it supplies how to read its config.json and how to describe its layers as a
:class:`ModelSpec` (parts chosen layer by layer); nothing else in the library
names a model.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .llama import ConfigError, MAX_CONFIG_BYTES, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]   # config.json dict -> typed config
    model_spec: Callable[[Any], Any]                        # typed config -> parts.spec.ModelSpec
    tolerated_extra_tensors: Callable[[str], bool] = lambda name: False


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, *, replace: bool = False) -> None:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name} is already registered")
    _ARCHITECTURES[arch.name] = arch


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"config: unsupported architecture {name}") from None


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def parse_config(text_or_dict) -> tuple[Architecture, Any]:
    """config.json (text or dict) -> (architecture entry, typed config)."""
    root = read_config_json(text_or_dict) if isinstance(text_or_dict, (str, bytes)) else dict(text_or_dict)
    arch = get_architecture(architecture_name(root))
    return arch, arch.config_from_dict(root)


def read_model_config(model_dir: str) -> tuple[Architecture, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        size = os.path.getsize(path)
    except OSError:
        raise ConfigError(f"cannot open {path}") from None
    if size > MAX_CONFIG_BYTES:
        raise ConfigError(f"{path} is larger than {MAX_CONFIG_BYTES} bytes")
    with open(path, "r", encoding="utf-8") as f:
        text = f.read()
    try:
        return parse_config(text)
    except ConfigError as e:
        raise ConfigError(f"{path}: {e}") from None
