"""One registry from an architecture's name to its configuration class.

``config.json`` names the architecture (``architectures[0]``, else ``model_type``);
the registered class reads the architecture's own keys and produces a ``ModelSpec``.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Mapping, Optional

from .spec import ConfigError, ModelSpec

# name -> callable(config_dict, generation_config_dict_or_None) -> object with .to_model_spec()
_ARCHITECTURES: Dict[str, Callable] = {}
_MODEL_TYPES: Dict[str, str] = {}


def register_architecture(name: str, config_class: Callable, model_type: Optional[str] = None) -> None:
    """Registers ``config_class.from_json(config, generation_config)`` under ``name``.

    ``model_type`` is the fallback key for a config.json that has no ``architectures``."""
    _ARCHITECTURES[name] = config_class
    if model_type:
        _MODEL_TYPES[model_type] = name


def registered_architectures():
    return sorted(_ARCHITECTURES)


def resolve_architecture(config: Mapping) -> str:
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)) and archs:
        name = archs[0]
        if name in _ARCHITECTURES:
            return name
        # fall through to model_type only if it is known; otherwise report the named architecture
        mt = config.get("model_type")
        if mt in _MODEL_TYPES:
            return _MODEL_TYPES[mt]
        raise ConfigError(
            f"unsupported architecture {name!r} (registered: {', '.join(registered_architectures())})")
    mt = config.get("model_type")
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    raise ConfigError(
        f"config.json names no known architecture (architectures={archs!r}, model_type={mt!r}); "
        f"registered: {', '.join(registered_architectures())}")


def config_from_dict(config: Mapping, generation_config: Optional[Mapping] = None):
    name = resolve_architecture(config)
    return _ARCHITECTURES[name].from_json(config, generation_config)


def load_config(model_dir: str):
    """Reads ``config.json`` (and ``generation_config.json`` if present) of a model folder."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{model_dir}: no config.json")
    with open(path, "r", encoding="utf-8") as f:
        config = json.load(f)
    gen = None
    gen_path = os.path.join(model_dir, "generation_config.json")
    if os.path.isfile(gen_path):
        with open(gen_path, "r", encoding="utf-8") as f:
            gen = json.load(f)
    return config_from_dict(config, gen)


def load_model_spec(model_dir: str) -> ModelSpec:
    return load_config(model_dir).to_model_spec()
