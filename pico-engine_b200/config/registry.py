"""The one registry from an architecture's name (``config.json["architectures"][0]``)
to its configuration class and the function that builds its model.

pico-engine chooses between its models with ``if`` chains on the file's metadata
(src/pico_engine/engine.py:28-30, src/pico_engine/model.py:140-145); here the choice is a
table, so that another architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict

from .specs import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type          # has from_dict(dict), to_dict() and plan() -> ModelPlan
    build_model: Callable       # (config, dtype, device) -> model


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_model: Callable | None = None) -> None:
    """Register ``name``.  With ``build_model`` None the model is the generic decoder
    assembled from ``config.plan()``."""
    if build_model is None:
        def build_model(config, dtype, device):
            from ..parts.model import DecoderModel
            return DecoderModel(config.plan(), dtype=dtype, device=device)
    _ARCHITECTURES[name] = Architecture(name, config_class, build_model)


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or 'none'}") from None


def architecture_name_of(config_dict: dict) -> str:
    archs = config_dict.get("architectures")
    if not isinstance(archs, (list, tuple)) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError(f'config.json needs "architectures": [one name]; found {archs!r}')
    return archs[0]


def config_from_dict(config_dict: dict):
    return architecture(architecture_name_of(config_dict)).config_class.from_dict(config_dict)


def read_config(folder: str):
    """The typed configuration of the model folder ``folder`` (its config.json)."""
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path, "r", encoding="utf-8") as f:
        return config_from_dict(json.load(f))
