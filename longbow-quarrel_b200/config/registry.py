"""One registry from an architecture's name (config.json `architectures[0]`) to its
typed configuration and to the function that describes its model from parts.

The reference keeps a registry of engine creators by backend name
(internal/engine/types_base.go:23-39); there is one backend here, so the registry
is by architecture instead.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict], Any]
    describe: Callable[[Any], Any]  # typed config -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, describe) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, describe)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_of(data: dict) -> Architecture:
    archs = data.get("architectures")
    if not archs or not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list that names the model class")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"config.json: architecture {name!r} is not registered "
                          f"(registered: {', '.join(registered_architectures()) or 'none'})")
    return _ARCHITECTURES[name]


def load_config(folder_or_file):
    """(architecture, typed config) of a model folder."""
    data = read_config_json(folder_or_file)
    arch = architecture_of(data)
    return arch, arch.config_from_dict(data)
