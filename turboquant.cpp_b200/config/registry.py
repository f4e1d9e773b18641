"""One registry from an architecture's name to its configuration and model.

config.json names the architecture in ``architectures[0]``; the registry maps
that name to the class that reads the rest of the file and to the class that
builds the model from it.  The reference selects model code by an integer
``model_type`` and substring tests on the GGUF architecture string
(src/engine/tq_model.c:3031-3056) and fails with a message when it finds no
supported layers (src/engine/tq_model.c:3822-3831); here an unknown name is
an error that lists the registered names.

Adding an architecture: write a config class with ``from_dict(raw, where)``,
a model class with ``__init__(config, dtype)`` (usually a subclass of
``models.decoder.DecoderModel`` that lists its blocks), and call
``register_architecture(name, ConfigClass, ModelClass)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Tuple

from .reader import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any
    model_class: Any


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, model_class: Any, replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _REGISTRY[name] = Architecture(name, config_class, model_class)


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def registered_architectures() -> Tuple[str, ...]:
    return tuple(sorted(_REGISTRY))


def architecture_name(raw: Dict[str, Any], where: str = "config.json") -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{where}: required key 'architectures' must be a non-empty list of names")
    return archs[0]


def lookup_architecture(name: str) -> Architecture:
    if name not in _REGISTRY:
        known = ", ".join(registered_architectures()) or "(none)"
        raise ConfigError(f"architecture '{name}' is not registered; registered: {known}")
    return _REGISTRY[name]


def parse_config(raw: Dict[str, Any], where: str = "config.json"):
    """Returns (Architecture, typed config) for a config.json dictionary."""
    arch = lookup_architecture(architecture_name(raw, where))
    return arch, arch.config_class.from_dict(raw, where)


def load_config(folder: str):
    raw = read_config_json(folder)
    return parse_config(raw, where=f"{folder}/config.json")
