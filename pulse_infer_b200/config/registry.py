"""One registry from the architecture's name (config.json ``architectures[0]``) to its model.

An architecture is a pair: the typed configuration class that reads config.json, and a builder
that turns a configuration into a ``ModelSpec`` (which parts, in which order, fed by which tensor
names).  The reference has no registry - its demos construct ``Qwen3Model`` directly
(``demo/qwen3_infer.cpp:612``) - so this is where a second architecture would plug in.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable

from .base import ConfigError, ModelConfig, read_json_file, resolve_model_dir


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable  # (config) -> ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable, model_type: str | None = None,
                          replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    arch = Architecture(name, config_class, build_spec)
    _ARCHITECTURES[name] = arch
    if model_type:
        _MODEL_TYPES[model_type] = name
    return arch


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(sorted(_ARCHITECTURES))}")
    return _ARCHITECTURES[name]


def architecture_name_of(obj: dict, source: str) -> str:
    _ensure_builtin()
    archs = obj.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    model_type = obj.get("model_type")
    if isinstance(model_type, str) and model_type in _MODEL_TYPES:
        return _MODEL_TYPES[model_type]
    if not archs and not model_type and len(_ARCHITECTURES) == 1:
        return next(iter(_ARCHITECTURES))      # the file names nothing and there is only one to choose from
    raise ConfigError(f"'{source}' names no architecture (key 'architectures'); known: "
                      f"{', '.join(sorted(_ARCHITECTURES))}")


def load_config(path: str) -> ModelConfig:
    """Read ``config.json`` of a model folder with the configuration class its architecture names."""
    model_dir = resolve_model_dir(path)
    config_path = os.path.join(model_dir, "config.json")
    obj = read_json_file(config_path)
    arch = get_architecture(architecture_name_of(obj, config_path))
    return arch.config_class.load(model_dir)


def _ensure_builtin() -> None:
    # importing the models package registers the architectures this framework ships
    from .. import models  # noqa: F401
