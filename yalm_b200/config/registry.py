"""The one registry from an architecture's name (``architectures[0]`` of
config.json) to its typed configuration class.  The reference routes its
supported names through one list (convert.py:15-19, 31); here each name maps
to a class with ``from_dict(config_json) -> cfg`` and ``cfg.to_spec()``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict

from .llama import ConfigError, LlamaConfig

_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_class: Any) -> None:
    """``config_class`` needs ``from_dict(dict)`` returning an object with
    ``to_spec() -> ModelSpec`` and ``to_dict() -> dict``."""
    _ARCHITECTURES[name] = config_class


def architectures() -> Dict[str, Any]:
    return dict(_ARCHITECTURES)


def config_from_dict(d: Dict[str, Any]) -> Any:
    archs = d.get("architectures")
    if not archs:
        raise ConfigError("config.json has no 'architectures' entry")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"architecture {name!r} is not registered; known: {sorted(_ARCHITECTURES)}")
    return _ARCHITECTURES[name].from_dict(d)


def load_config(model_dir: str) -> Any:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {model_dir}")
    with open(path, "r") as f:
        return config_from_dict(json.load(f))


register_architecture("LlamaForCausalLM", LlamaConfig)
register_architecture("MistralForCausalLM", LlamaConfig)
