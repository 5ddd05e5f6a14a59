"""One registry from an architecture's name (config.json `architectures[0]`)
to its configuration class and the function that puts its model together.

The reference's table of supported architectures is
`SUPPORTED_ARCHES` (alpacca/model.py:22-29) with the rejection at :189-193.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Callable

from .base import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build: Callable  # (config, BuildOptions) -> DecoderSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type):
    """Decorator: `@register_architecture("XForCausalLM", XConfig) def build(cfg, opts): ...`"""
    def deco(build):
        if name in _ARCHITECTURES:
            raise ValueError(f"architecture {name!r} is registered twice")
        _ARCHITECTURES[name] = Architecture(name, config_class, build)
        return build
    return deco


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture {name!r} is not supported "
                          f"(supported: {', '.join(sorted(_ARCHITECTURES)) or 'none'})") from None


def config_from_dict(d: dict) -> ModelConfig:
    """Picks the configuration class by `architectures[0]` and reads the keys with it."""
    archs = d.get("architectures")
    name = d.get("architecture") or (archs[0] if isinstance(archs, list) and archs else None)
    if not name:
        raise ConfigError("config.json has no 'architectures' entry")
    return get_architecture(name).config_class.from_dict(d)


def load_config(model_dir) -> ModelConfig:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise ConfigError(f"no config.json in {model_dir}")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return config_from_dict(d)


def _load_builtin() -> None:
    # the built-in architectures register themselves on import
    from .. import models  # noqa: F401
