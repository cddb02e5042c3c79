"""Typed model configurations and the registry from architecture name to model.

A configuration class owns the reading of one architecture's config.json keys; no
size or constant that config.json gives stands anywhere else in the package.  The
registry maps the name found in config.json's `architectures[0]` (or `model_type`,
the reference's fallback: src/convert/hf.zig:229-234) to a configuration class and a
function that builds the model description from it.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, Tuple


class ConfigError(ValueError):
    """A config.json key is missing, malformed or names something unsupported.
    The message names the key and the value (cf. `Diag`, src/engine/config.zig:104-116)."""


@dataclass
class ModelConfig:
    """Base of every architecture's typed configuration."""

    architecture: str

    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        """config.json content that `from_dict` reads back to an equal object."""
        raise NotImplementedError


_REGISTRY: Dict[str, Tuple[type, Callable]] = {}


def register_architecture(name: str, config_cls: type, build_model: Callable, *aliases: str) -> None:
    """Registers `build_model(config) -> ModelSpec` under `name` (and aliases)."""
    for n in (name, *aliases):
        _REGISTRY[n] = (config_cls, build_model)


def supported_architectures():
    return sorted(_REGISTRY)


def resolve_architecture(name: str):
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(
            f"architecture '{name}' is not supported (supported: {', '.join(supported_architectures())})"
        ) from None


def architecture_name(raw: dict) -> str:
    archs = raw.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    mt = raw.get("model_type")
    if isinstance(mt, str):
        return mt
    raise ConfigError("config.json names no architecture (neither 'architectures' nor 'model_type')")


def load_config(model_dir: str) -> ModelConfig:
    """Reads `<model_dir>/config.json` into the typed configuration of its architecture."""
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"no config.json in '{model_dir}'") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} does not hold a JSON object")
    return config_from_dict(raw)


def config_from_dict(raw: dict) -> ModelConfig:
    config_cls, _ = resolve_architecture(architecture_name(raw))
    return config_cls.from_dict(raw)


# ---- helpers for configuration classes -------------------------------------------------


def need_int(raw: dict, key: str, minimum: int = 1) -> int:
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json has no '{key}'")
    return _as_int(raw[key], key, minimum)


def opt_int(raw: dict, key: str, default, minimum: int = 1):
    v = raw.get(key)
    if v is None:
        return default
    return _as_int(v, key, minimum)


def _as_int(v, key: str, minimum: int) -> int:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        raise ConfigError(f"config.json '{key}' = {v!r} is not a whole number")
    v = int(v)
    if v < minimum:
        raise ConfigError(f"config.json '{key}' = {v} is below {minimum}")
    return v


def opt_float(raw: dict, key: str, default: float) -> float:
    v = raw.get(key)
    if v is None:
        return float(default)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json '{key}' = {v!r} is not a number")
    return float(v)


def opt_bool(raw: dict, key: str, default: bool) -> bool:
    v = raw.get(key)
    if v is None:
        return default
    if not isinstance(v, bool):
        raise ConfigError(f"config.json '{key}' = {v!r} is not true or false")
    return v
