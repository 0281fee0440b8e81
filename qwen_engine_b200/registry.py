"""One registry from an architecture's name (``config.json``'s
``architectures[0]``) to its configuration class and its layout function.

The reference has no registry: its ``models/__init__.py`` re-exports the one
model it has (src/models/__init__.py:1-3).  Another architecture is added with
``register_architecture(name, ConfigClass, layout_fn)``; the engine, the loader
and the cache manager ask the model that comes out, not the architecture.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .config import ConfigError, ModelConfig, Qwen3Config, read_config_json
from .models.decoder import DecoderModel, ModelLayout
from .models.qwen3 import qwen3_layout


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    layout: Callable[[Any], ModelLayout]


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, layout: Callable[[Any], ModelLayout]) -> None:
    ARCHITECTURES[name] = Architecture(name, config_class, layout)


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_layout)


def architecture_of(raw_config: dict[str, Any]) -> Architecture:
    names = raw_config.get("architectures")
    if not names or not isinstance(names, list):
        raise ConfigError("config.json: 'architectures' is missing; known: "
                          f"{sorted(ARCHITECTURES)}")
    if names[0] not in ARCHITECTURES:
        raise ConfigError(f"config.json: architecture {names[0]!r} is not registered; known: "
                          f"{sorted(ARCHITECTURES)}")
    return ARCHITECTURES[names[0]]


def config_from_dict(raw_config: dict[str, Any]) -> ModelConfig:
    return architecture_of(raw_config).config_class.from_dict(raw_config)


def config_from_folder(model_dir: str) -> ModelConfig:
    return config_from_dict(read_config_json(model_dir))


def build_model(config: ModelConfig) -> DecoderModel:
    arch = ARCHITECTURES.get(config.architecture)
    if arch is None:
        raise ConfigError(f"architecture {config.architecture!r} is not registered")
    return DecoderModel(arch.layout(config))


def weight_manifest_for(config: ModelConfig):
    return build_model(config).weight_manifest()
