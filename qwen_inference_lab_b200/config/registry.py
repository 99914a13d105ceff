"""The one table from an architecture's name to its configuration class and builder.

``config.json`` names the architecture in ``architectures[0]`` (falling back to
``model_type``); everything else in the engine asks this table and never a model
class directly.  The reference has no such table: it refuses every ``model_type``
but ``qwen3`` in place (qil/config.py:37-38).  Adding an architecture is one
``register`` call with a configuration class (``from_dict``/``to_dict``) and a
function ``build(config) -> DecoderModel``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    model_type: str
    config_class: type
    build: Callable


_by_name: dict = {}
_by_model_type: dict = {}


def register(name, model_type, config_class, build) -> Architecture:
    if name in _by_name:
        raise ValueError(f"architecture {name} is already registered")
    entry = Architecture(name, model_type, config_class, build)
    _by_name[name] = entry
    _by_model_type.setdefault(model_type, entry)
    return entry


def unregister(name) -> None:
    entry = _by_name.pop(name, None)
    if entry is not None and _by_model_type.get(entry.model_type) is entry:
        del _by_model_type[entry.model_type]


def known() -> list:
    return sorted(_by_name)


def lookup(config_dict: dict) -> Architecture:
    names = config_dict.get("architectures") or []
    if names:
        entry = _by_name.get(names[0])
        if entry is None:
            raise ConfigError(f"architecture {names[0]!r} is not supported (known: {known()})")
        return entry
    entry = _by_model_type.get(config_dict.get("model_type"))
    if entry is None:
        raise ConfigError(
            f"config.json names no architecture and model_type {config_dict.get('model_type')!r} "
            f"is unknown (known architectures: {known()})")
    return entry


def read_model_config(directory):
    """(architecture entry, typed configuration) of a model folder."""
    data = read_config_json(directory)
    entry = lookup(data)
    return entry, entry.config_class.from_dict(data)
