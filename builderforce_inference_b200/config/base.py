"""Typed reading of a ``config.json`` dictionary.

A configuration class reads every size and constant of its architecture through a
``ConfigReader``; a key that is missing, of the wrong type or out of range becomes a
``ConfigError`` that names the key, so a bad folder fails before any weight is read.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Iterable, Optional


class ConfigError(ValueError):
    """A config.json key is missing, mistyped, out of range or asks for an unsupported option."""


_MISSING = object()


class ConfigReader:
    """Reads typed values out of a config.json dictionary and remembers which keys were used."""

    def __init__(self, data: Dict[str, Any], what: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{what}: expected a JSON object, got {type(data).__name__}")
        self.data = data
        self.what = what
        self.used: set = set()

    def has(self, key: str) -> bool:
        return key in self.data and self.data[key] is not None

    def raw(self, key: str, default: Any = None) -> Any:
        self.used.add(key)
        v = self.data.get(key, default)
        return default if v is None else v

    def _get(self, key: str, default: Any) -> Any:
        self.used.add(key)
        v = self.data.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.what}: missing required key '{key}'")
            return default
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> Any:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v == int(v):
                v = int(v)
            else:
                raise ConfigError(f"{self.what}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.what}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> Any:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.what}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.what}: key '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, bool):
            raise ConfigError(f"{self.what}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, str):
            raise ConfigError(f"{self.what}: key '{key}' must be a string, got {v!r}")
        return v

    def string_list(self, key: str, default: Any = _MISSING) -> Any:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if not isinstance(v, (list, tuple)) or not all(isinstance(s, str) for s in v):
            raise ConfigError(f"{self.what}: key '{key}' must be a list of strings, got {v!r}")
        return list(v)

    def int_or_list(self, key: str) -> Iterable[int]:
        """An id or a list of ids (``eos_token_id`` comes both ways); absent gives ``()``."""
        v = self._get(key, ())
        if isinstance(v, bool):
            raise ConfigError(f"{self.what}: key '{key}' must be an integer or a list of them")
        if isinstance(v, int):
            return (v,)
        if isinstance(v, (list, tuple)) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return tuple(v)
        raise ConfigError(f"{self.what}: key '{key}' must be an integer or a list of them, got {v!r}")


def read_json(path: str) -> Dict[str, Any]:
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path, "r", encoding="utf-8") as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from e


def stop_ids_of_folder(folder: str, from_config: Iterable[int]) -> tuple:
    """The stop token ids of a model folder: those of ``generation_config.json`` (key
    ``eos_token_id``, an id or a list) when that file is there, followed by the ones config.json
    names that it does not repeat; config.json's alone otherwise.  The reference takes its end
    token from the model file's metadata as well (crates/bfi-runtime/src/tokenize.rs:68)."""
    ids = list(from_config)
    path = os.path.join(folder, "generation_config.json")
    if os.path.isfile(path):
        first = list(ConfigReader(read_json(path), path).int_or_list("eos_token_id"))
        ids = first + [i for i in ids if i not in first]
    return tuple(ids)
