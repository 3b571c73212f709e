"""The one registry from an architecture's name (config.json ``architectures[0]``)
to its typed configuration and its model.

berniehans/titan has no registry: ``ForwardDriver`` serves the dense family and
switches on tensor presence (engine/engine-core/src/forward_driver.rs:628-629).
Here the name decides, everywhere: loader, engine, replay and command line all
come through ``load_config``.

An entry is a configuration class with ``from_dict(dict)`` and
``to_model_spec() -> ModelSpec``.  The model itself is always assembled from the
``ModelSpec`` by the part registries, so adding an architecture is: write its
configuration class, and register it here (or from outside the package with
``register_architecture``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict

from .spec import ConfigError

_ARCHITECTURES: Dict[str, Any] = {}


def register_architecture(name: str, config_class: Any) -> None:
    if not (hasattr(config_class, "from_dict") and hasattr(config_class, "to_model_spec")):
        raise TypeError("a configuration class needs from_dict(dict) and to_model_spec()")
    _ARCHITECTURES[name] = config_class


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_from_dict(d: Dict[str, Any]):
    archs = d.get("architectures")
    if not archs or not isinstance(archs, list):
        raise ConfigError("config.json lacks the key 'architectures'")
    name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not registered; known: {', '.join(known_architectures())}")
    return _ARCHITECTURES[name].from_dict(d)


def load_config(model_dir: str):
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {model_dir}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None
    return config_from_dict(d)
