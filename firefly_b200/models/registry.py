"""The one registry from an architecture's name to its model.

An architecture is registered as a pair: its typed configuration class and a
function that turns such a configuration into a ``ModelSpec`` (the model as
data).  The generic decoder in ``models/decoder.py`` builds and runs any spec.
The reference keeps the same kind of map from ``config.json``'s
``architectures[0]`` to a factory (src/model_registry.cc:14-27,
src/model/qwen_model.cu:195-207) and throws "Unknown model architecture" for a
name it does not hold.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Tuple, Type

from ..config.base import ConfigError, ModelConfig, ModelSpec, read_config_json

_ARCHITECTURES: Dict[str, Tuple[Type[ModelConfig], Callable[[ModelConfig], ModelSpec]]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          spec_builder: Callable[[ModelConfig], ModelSpec], *,
                          replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = (config_cls, spec_builder)


def known_architectures():
    return sorted(_ARCHITECTURES)


def _entry(name: str):
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown model architecture '{name}'; known: "
                          f"{', '.join(known_architectures()) or '(none)'}") from None


def architecture_of(raw: Mapping[str, Any]) -> str:
    archs = raw.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
    return archs[0]


def config_from_dict(raw: Mapping[str, Any]) -> ModelConfig:
    """Typed configuration for whatever architecture ``raw`` names."""
    cls, _ = _entry(architecture_of(raw))
    return cls.from_dict(raw)


def load_config(model_dir: str) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


def spec_for(config: ModelConfig) -> ModelSpec:
    _, builder = _entry(config.architecture)
    return builder(config)
