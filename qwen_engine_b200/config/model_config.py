"""Typed model configurations read from a model folder's ``config.json``.

Every size and constant of a model comes from the keys of its own
``config.json``; nothing in the code stands in for them.  This file holds what
every architecture shares: the base class, the error type, reading and writing
of ``config.json``.  An architecture's own dataclass lives in a file of its own
(``qwen3_config.py``).
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, ClassVar, Optional


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses are dataclasses whose field names are the ``config.json`` keys.
    ``architecture`` names the registry entry that builds the model.
    """

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that reads back as this configuration."""
        out = dataclasses.asdict(self)
        out["architectures"] = [self.architecture]
        return out

    def validate(self) -> None:
        raise NotImplementedError


def _require_int(name: str, value: Any, minimum: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ConfigError(f"config.json: {name} must be an integer, got {value!r}")
    if value < minimum:
        raise ConfigError(f"config.json: {name} must be >= {minimum}, got {value}")
    return value


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def write_config_json(config: ModelConfig, model_dir: str) -> str:
    os.makedirs(model_dir, exist_ok=True)
    path = os.path.join(model_dir, "config.json")
    with open(path, "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2, sort_keys=True)
        f.write("\n")
    return path
