"""The one table from an architecture's name (``architectures[0]`` of config.json) to its
typed configuration and its model specification.

The reference picks a class with if/else on substrings and on
``num_hidden_layers / num_key_value_heads == 16`` (cpmcu/common/utils.py:33-64, 147-162).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Tuple

from .config.base import ConfigError, architecture_name, read_config_json
from .parts.base import ModelSpec


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                                   # has from_dict(dict) and to_dict()
    model_spec: Callable[[Any], ModelSpec]              # typed config -> specification
    adapt_tensor: Optional[Callable[[Any, str, Any], List[Tuple[str, Any]]]] = None
    ignore_tensor: Optional[Callable[[str], bool]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


_plugins_loaded: set = set()


def load_plugins(modules=None) -> List[str]:
    """Imports the named modules (default: the comma-separated list in the environment variable
    ``CPMCU_PLUGINS``), each once.  A plug-in is any importable module that registers parts or architectures when
    it is imported; this is how a model that the package does not know is reached from the command line and
    from ``bin/trace_run`` without a change to the package."""
    import importlib
    import os

    if modules is None:
        modules = [m.strip() for m in os.environ.get("CPMCU_PLUGINS", "").split(",") if m.strip()]
    done = []
    for m in modules:
        if m not in _plugins_loaded:
            _plugins_loaded.add(m)
            importlib.import_module(m)
            done.append(m)
    return done


def architecture(name: str) -> Architecture:
    load_plugins()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; known: {sorted(_ARCHITECTURES)}") from None


def known_architectures() -> List[str]:
    load_plugins()
    return sorted(_ARCHITECTURES)


def load_config(model_dir: str):
    """(architecture, typed configuration) of a model folder."""
    data = read_config_json(model_dir)
    arch = architecture(architecture_name(data))
    return arch, arch.config_class.from_dict(data)


def _register_builtin() -> None:
    from .config.minicpm import MiniCPMConfig
    from .models import minicpm4

    register_architecture(Architecture(
        name="MiniCPMForCausalLM",
        config_class=MiniCPMConfig,
        model_spec=minicpm4.model_spec,
        adapt_tensor=minicpm4.split_fused_tensors,
        ignore_tensor=minicpm4.ignored_tensor,
    ))


_register_builtin()
