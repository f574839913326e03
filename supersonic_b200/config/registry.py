"""One registry from an architecture's name to its configuration class.

``config.json``'s ``architectures[0]`` picks the entry, everywhere in the
framework.  The reference maps CLI aliases to a family enum and dispatches with
a ``match`` (crates/runner/src/registry.rs:41-59, main.rs:1401-1413); here the
table is open: adding an architecture is one ``register_architecture`` call
with a class that offers ``from_dict``, ``to_dict``, ``build_spec`` and
``tensor_shapes``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .base import ConfigError, ModelSpec
from .llama import ARCHITECTURE as _LLAMA, LlamaConfig

_ARCHITECTURES: Dict[str, Type] = {}


def register_architecture(name: str, config_cls: Type) -> None:
    for attr in ("from_dict", "to_dict", "build_spec", "tensor_shapes"):
        if not hasattr(config_cls, attr):
            raise TypeError(f"{config_cls.__name__} lacks {attr}()")
    _ARCHITECTURES[name] = config_cls


def known_architectures():
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str) -> Type:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {known_architectures()}") from None


def config_from_dict(d: Dict[str, Any]):
    archs = d.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json has no 'architectures' list")
    return lookup_architecture(archs[0]).from_dict(d)


def load_config(model_dir: str):
    """Read ``config.json`` of a model folder into its typed configuration."""
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except OSError as e:
        raise ConfigError(f"read config.json: {e}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"parse config.json: {e}") from None
    return config_from_dict(d)


def spec_from_config(config) -> ModelSpec:
    return config.build_spec()


register_architecture(_LLAMA, LlamaConfig)


_PRESET_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "presets")


def preset_names():
    """Named sizes for random-weight runs: one config.json-shaped file each."""
    return sorted(f[:-5] for f in os.listdir(_PRESET_DIR) if f.endswith(".json"))


def preset_config(name: str, **overrides):
    path = os.path.join(_PRESET_DIR, name + ".json")
    if not os.path.isfile(path):
        raise ConfigError(f"unknown preset {name!r}; known: {preset_names()}")
    with open(path, "r", encoding="utf-8") as f:
        d = json.load(f)
    d.update(overrides)
    return config_from_dict(d)
