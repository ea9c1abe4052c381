"""Typed model configuration: the base class and the JSON helpers every architecture shares.

A configuration is a frozen dataclass whose fields are exactly the keys of the architecture's own
``config.json``.  No size lives anywhere else: parts receive their sizes and constants from the
configuration through the architecture's builder (``pulse_infer_b200.models``).

Reference parity: ``src/model/qwen3/config.cpp:70-138`` (typed key readers with one error message
per missing or mistyped key) and ``config.cpp:231-239`` (a path may name the folder or a file in it).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type, or a value out of range."""


def resolve_model_dir(path: str) -> str:
    """Accept a model folder or any file inside it (config.cpp:38-44)."""
    path = os.fspath(path)
    if os.path.isdir(path):
        return path
    parent = os.path.dirname(os.path.abspath(path))
    if os.path.isfile(path) and os.path.isdir(parent):
        return parent
    raise ConfigError(f"model path '{path}' is neither a folder nor a file inside one")


def read_json_file(path: str) -> dict:
    if not os.path.isfile(path):
        raise ConfigError(f"Config file '{path}' does not exist")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            obj = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"Config file '{path}' is not valid JSON: {exc}") from exc
    if not isinstance(obj, dict):
        raise ConfigError(f"Config file '{path}' must hold a JSON object")
    return obj


class KeyReader:
    """Typed access to one JSON object; every failure names the key, the wanted type and the file."""

    def __init__(self, obj: dict, source: str):
        self.obj = obj
        self.source = source

    def _fail(self, kind: str, key: str) -> ConfigError:
        return ConfigError(f"Missing or invalid {kind} key '{key}' in '{self.source}'")

    def has(self, key: str) -> bool:
        return key in self.obj and self.obj[key] is not None

    def int(self, key: str, default: Any = ...) -> int:
        if not self.has(key):
            if default is ...:
                raise self._fail("integer", key)
            return default
        v = self.obj[key]
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                return int(v)
            raise self._fail("integer", key)
        return v

    def float(self, key: str, default: Any = ...) -> float:
        if not self.has(key):
            if default is ...:
                raise self._fail("float", key)
            return default
        v = self.obj[key]
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise self._fail("float", key)
        return float(v)

    def bool(self, key: str, default: Any = ...) -> bool:
        if not self.has(key):
            if default is ...:
                raise self._fail("boolean", key)
            return default
        v = self.obj[key]
        if not isinstance(v, bool):
            raise self._fail("boolean", key)
        return v

    def str(self, key: str, default: Any = ...) -> str:
        if not self.has(key):
            if default is ...:
                raise self._fail("string", key)
            return default
        v = self.obj[key]
        if not isinstance(v, str):
            raise self._fail("string", key)
        return v

    def int_list(self, key: str) -> tuple:
        """An integer or a list of integers; absent gives an empty tuple (config.cpp:140-176)."""
        if not self.has(key):
            return ()
        v = self.obj[key]
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return tuple(v)
        raise self._fail("integer-or-list", key)

    def str_list(self, key: str) -> tuple | None:
        if not self.has(key):
            return None
        v = self.obj[key]
        if isinstance(v, list) and all(isinstance(x, str) for x in v):
            return tuple(v)
        raise self._fail("string-list", key)


@dataclass(frozen=True)
class ModelConfig:
    """Fields every architecture's configuration carries.  ``architecture`` selects the model class."""

    architecture: str

    def to_json_dict(self) -> dict:
        """The config.json this configuration is read back from (used by the random-weights mode)."""
        raise NotImplementedError
