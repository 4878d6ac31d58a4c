"""One registry from an architecture's name to its configuration class and model builder.

The reference serves one model and has no registry; this engine keys everything on
`architectures[0]` of config.json. An entry names the typed configuration class that
reads config.json, the manifest of tensor names and shapes the architecture expects, and a
builder that turns (configuration, weights) into a `ModelSpec` of parts. Unknown names fail with the list of known ones.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from ..errors import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type                 # has from_dict(dict, where) and to_dict()
    manifest: Callable               # manifest(config) -> {tensor name: TensorSpec}
    build: Callable                  # build(config, weights: WeightSet, ctx: BuildContext) -> ModelSpec


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> None:
    if arch.name in _REGISTRY and not replace:
        raise ConfigError(f"architecture {arch.name!r} is already registered")
    _REGISTRY[arch.name] = arch


def unregister_architecture(name: str) -> None:
    _REGISTRY.pop(name, None)


def known_architectures():
    return sorted(_REGISTRY)


def architecture_for(config_dict: dict, where: str = "config.json") -> Architecture:
    archs = config_dict.get("architectures")
    if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
        raise ConfigError(f"{where}: 'architectures' must be a list with the model class name")
    try:
        return _REGISTRY[archs[0]]
    except KeyError:
        raise ConfigError(f"{where}: architecture {archs[0]!r} is not known; known: "
                          f"{', '.join(known_architectures()) or '(none)'}") from None
