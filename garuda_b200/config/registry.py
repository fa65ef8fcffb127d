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


def load_plugins(names=None) -> None:
    """Imports modules that register architectures or parts of their own (each calls
    ``register_architecture`` / ``register_mixer`` / ... when imported). ``names``: module names;
    those of the environment variable ``GARUDA_B200_PLUGINS`` (comma separated) are imported as
    well. The command line's ``--plugin`` and a config.toml's ``[model] plugins`` end up here."""
    import importlib
    import os
    wanted = list(names or [])
    wanted += [n for n in os.environ.get("GARUDA_B200_PLUGINS", "").split(",") if n.strip()]
    for name in wanted:
        try:
            importlib.import_module(name.strip())
        except ImportError as e:
            raise ConfigError(f"plugin module '{name}' cannot be imported: {e}") from None


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
