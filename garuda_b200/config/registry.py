"""One registry from an architecture's name to its configuration class and model.

The reference dispatches on the checkpoint's ``general.architecture`` string
(garuda/src/server/mod.rs:372-377) and refuses what it does not know
(garuda/src/llama/mod.rs:415-420). Here the key is ``architectures[0]`` of
config.json. An architecture is added with ``register_architecture(name,
read_config, make_spec)``: ``read_config`` turns the config.json dictionary
into a typed configuration, ``make_spec`` turns that into a ``ModelSpec``.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .model_config import ConfigError

_ARCHITECTURES: Dict[str, Tuple[Callable, Callable]] = {}


def register_architecture(name: str, read_config: Callable, make_spec: Callable) -> None:
    _ARCHITECTURES[name] = (read_config, make_spec)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def architecture_of(config_dict: dict) -> str:
    archs = config_dict.get("architectures")
    if not archs:
        raise ConfigError("config.json is missing 'architectures'")
    return archs[0]


def read_model_config(config_dict: dict):
    """Typed configuration of whatever architecture the dictionary names."""
    name = architecture_of(config_dict)
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture '{name}' is not supported "
                          f"(registered: {', '.join(registered_architectures()) or 'none'})")
    return _ARCHITECTURES[name][0](config_dict)


def build_model(config_dict: dict):
    """(typed configuration, Decoder without weights) for a config.json dictionary."""
    from ..models.decoder import Decoder
    name = architecture_of(config_dict)
    cfg = read_model_config(config_dict)
    return cfg, Decoder(_ARCHITECTURES[name][1](cfg))
