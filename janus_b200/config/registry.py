"""One registry from an architecture's name (config.json `architectures[0]`)
to its typed configuration and its model builder.

The reference keeps an allow-list of names that all run the same Llama code
(crates/janus-engine/src/model/config.rs:183-204) and reports the list on a
miss (config.rs:30-31).  Here each name owns an entry; only what is registered
is accepted.
"""
from __future__ import annotations

import importlib
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List

from .base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                 # has from_dict(dict) -> typed config
    build: Callable[..., Any]         # build(config, dtype, device) -> engine.model.DecoderModel (no weights yet)
    weight_specs: Callable[[Any], Any]  # weight_specs(config) -> list of weights.loader.TensorSpec


_REGISTRY: Dict[str, Architecture] = {}
DEFAULT_ARCHITECTURE = "LlamaForCausalLM"


def register_architecture(name: str, config_class: Any, build: Callable[..., Any],
                          weight_specs: Callable[[Any], Any]) -> None:
    _REGISTRY[name] = Architecture(name, config_class, build, weight_specs)


def registered_architectures() -> List[str]:
    _load_builtin()
    return sorted(_REGISTRY)


def _load_builtin() -> None:
    # Importing the package of models registers the built-in architectures; modules named in JANUS_PLUGINS
    # (comma-separated, importable names) are imported after it, so that the command line and the replay
    # program also serve architectures and parts that such a module registers.
    from .. import models  # noqa: F401
    for name in os.environ.get("JANUS_PLUGINS", "").split(","):
        if name.strip():
            importlib.import_module(name.strip())


def architecture_name(config_dict: Dict[str, Any]) -> str:
    """`architectures[0]`; a config without the key is taken as Llama, which
    the reference accepts too (config.rs:183)."""
    archs = config_dict.get("architectures")
    if archs is None or archs == []:
        return DEFAULT_ARCHITECTURE
    if not isinstance(archs, list) or not isinstance(archs[0], str):
        raise ConfigError(f"key 'architectures' must be a list of strings, got {archs!r}")
    return archs[0]


def resolve_architecture(config_dict: Dict[str, Any]) -> Architecture:
    _load_builtin()
    name = architecture_name(config_dict)
    entry = _REGISTRY.get(name)
    if entry is None:
        raise ConfigError(
            f"unsupported architecture '{name}'; registered: {', '.join(sorted(_REGISTRY))}")
    return entry
