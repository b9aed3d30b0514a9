"""Typed model configurations and the registry from architecture name to model.

A configuration class owns the reading of its architecture's ``config.json``
keys (names, defaults, what is refused) and nothing else.  The registry maps the
name in ``architectures[0]`` to a configuration class and to a function that
turns such a configuration into a ``ModelSpec`` (see ``kllm_b200.parts.spec``).
The reference has no registry: a two-valued ``arch`` integer is chosen by a prefix
of ``model_type`` (models/config.go:152-153; backend/model.cu:734-735).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Tuple


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the reason."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of all typed configurations."""

    architecture: str

    @classmethod
    def from_dict(cls, d: dict) -> "ModelConfig":  # pragma: no cover - interface
        raise NotImplementedError

    def to_dict(self) -> dict:  # pragma: no cover - interface
        raise NotImplementedError


_REGISTRY: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable) -> None:
    """Make ``name`` (as it stands in ``architectures``) known.

    ``config_cls.from_dict(dict)`` parses config.json; ``build_spec(config)``
    returns the ``ModelSpec`` from which the model is assembled.
    """
    _REGISTRY[name] = (config_cls, build_spec)


def known_architectures():
    return sorted(_REGISTRY)


def lookup_architecture(name: str):
    if name not in _REGISTRY:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures()) or '(none)'}")
    return _REGISTRY[name]


def parse_config(d: dict) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    config_cls, _ = lookup_architecture(archs[0])
    return config_cls.from_dict(d)


def load_config(model_dir: str) -> ModelConfig:
    """Read ``<model_dir>/config.json`` into its typed configuration
    (role of LoadConfig, models/config.go:102-125)."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"parsing {path}: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level is not an object")
    return parse_config(d)


def build_model_spec(config: ModelConfig):
    _, build_spec = lookup_architecture(config.architecture)
    return build_spec(config)


# ---- helpers for configuration classes ---------------------------------------

def take_int(d: dict, key: str, default=None, minimum=None) -> int:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: '{key}' is required")
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
    v = int(v)
    if minimum is not None and v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, got {v}")
    return v


def take_float(d: dict, key: str, default=None) -> float:
    v = d.get(key, default)
    if v is None:
        raise ConfigError(f"config.json: '{key}' is required")
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
    return float(v)
