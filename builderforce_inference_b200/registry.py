"""One registry from an architecture's name to its model.

A config.json names its architecture twice: ``architectures[0]`` (a class name such as
``Qwen3ForCausalLM``) and ``model_type`` (``qwen3``).  Either selects the entry; the lookup is
exact and case-sensitive, and an unknown name is answered with the list of known ones, as in
the reference (crates/bfi-models/src/arch.rs:70-91).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Tuple

from .config.base import ConfigError
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    describe: Callable[[Dict[str, Any]], ModelSpec]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(names: Tuple[str, ...], arch: Architecture) -> None:
    for n in names:
        if n in _ARCHITECTURES and _ARCHITECTURES[n] is not arch:
            raise ValueError(f"architecture name '{n}' is already registered")
        _ARCHITECTURES[n] = arch


def unregister_architecture(*names: str) -> None:
    for n in names:
        _ARCHITECTURES.pop(n, None)


def registered_architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def architecture_for(config: Dict[str, Any]) -> Architecture:
    candidates: List[str] = []
    archs = config.get("architectures")
    if isinstance(archs, (list, tuple)):
        candidates += [a for a in archs if isinstance(a, str)]
    if isinstance(config.get("model_type"), str):
        candidates.append(config["model_type"])
    if not candidates:
        raise ConfigError("config.json names no architecture (keys 'architectures' and 'model_type'); "
                          f"registered: {registered_architectures()}")
    for c in candidates:
        if c in _ARCHITECTURES:
            return _ARCHITECTURES[c]
    raise ConfigError(f"unsupported architecture '{candidates[0]}'; registered: {registered_architectures()}")


def describe_model(config: Dict[str, Any]) -> ModelSpec:
    return architecture_for(config).describe(config)


def _register_builtin() -> None:
    from .architectures import qwen3
    from .config.qwen3 import Qwen3Config
    register_architecture(("qwen3", "Qwen3ForCausalLM"),
                          Architecture(name="qwen3", config_class=Qwen3Config, describe=qwen3.describe))


_register_builtin()
