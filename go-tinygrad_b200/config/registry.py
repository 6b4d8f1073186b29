"""One registry from an architecture's name to what builds its model.

An entry names the configuration class that reads the architecture's own
config.json keys and a function that turns that configuration into a model
plan (the list of layers, the order they run in, and what each is made of).
The reference has no registry: one loader tests ``ModelType`` strings all
through its code (model/llama.go:257-262 and the ``if cfg.ModelType ==``
branches in :1094-1455); its own refactor notes call that out.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping, Tuple

from .llama import ConfigError


@dataclass(frozen=True)
class Architecture:
    """`names` are matched against config.json's ``architectures`` entries and
    ``model_type``.  `read_config(raw_json) -> config`; `plan(config) -> ModelPlan`.
    `ignore`: shell-style patterns of tensor names a checkpoint of this
    architecture may carry that no part reads (stored buffers and the like); a
    tensor that neither a part declares nor a pattern matches is still an error."""
    names: Tuple[str, ...]
    read_config: Callable[[Mapping[str, Any]], Any]
    plan: Callable[[Any], Any]
    ignore: Tuple[str, ...] = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> Architecture:
    for name in arch.names:
        if name in _ARCHITECTURES and not replace and _ARCHITECTURES[name] is not arch:
            raise ValueError(f"architecture name {name!r} is already registered")
    for name in arch.names:
        _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(arch: Architecture) -> None:
    for name in arch.names:
        if _ARCHITECTURES.get(name) is arch:
            del _ARCHITECTURES[name]


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def find_architecture(raw: Mapping[str, Any]) -> Architecture:
    """The entry for a parsed config.json: ``architectures`` first, then ``model_type``."""
    candidates = []
    archs = raw.get("architectures")
    if isinstance(archs, (list, tuple)):
        candidates += [str(a) for a in archs]
    if raw.get("model_type"):
        candidates.append(str(raw["model_type"]))
    if not candidates:
        raise ConfigError("config.json names no architecture: it has neither "
                          "'architectures' nor 'model_type'")
    for name in candidates:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    raise ConfigError(f"no registered architecture matches {candidates}; "
                      f"registered: {list(registered_architectures())}")


def read_config_json(folder: str) -> Mapping[str, Any]:
    path = os.path.join(folder, "config.json")
    try:
        with open(path) as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path} does not exist") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw


def read_model_config(folder: str):
    """(architecture entry, typed configuration) of a model folder."""
    raw = read_config_json(folder)
    arch = find_architecture(raw)
    return arch, arch.read_config(raw)
