"""Typed model configuration and the architecture registry.

A configuration class reads the keys its architecture writes to ``config.json``
and nothing else; every size the engine uses comes from an instance of it.  The
registry maps the name in ``config.json``'s ``architectures`` to (configuration
class, model builder), the way mischief/lgml maps a gguf architecture to its
family flags and module (``lua/lgml/transformer.lua:61-78``, ``:99``,
``lua/lgml/engine.lua:489``); an unknown name is an error that names it
(``lua/lgml/transformer.lua:125-127``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Any, Callable, Dict, Tuple, Type


class ConfigError(ValueError):
    """A config.json that the architecture cannot run; the message names the key."""


@dataclass
class ModelConfig:
    """Base of every architecture's configuration."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> Dict[str, Any]:
        raise NotImplementedError

    def validate(self) -> None:
        raise NotImplementedError

    def flat(self) -> Dict[str, Any]:
        """Scalars only, for logs and benchmark records."""
        out = {}
        for f in fields(self):
            v = getattr(self, f.name)
            if isinstance(v, (int, float, str, bool)) or v is None:
                out[f.name] = v
        return out


_REGISTRY: Dict[str, Tuple[Type[ModelConfig], Callable[..., Any]]] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig], builder: Callable[..., Any]) -> None:
    """Make ``name`` (as written in ``architectures``) loadable.  ``builder(config,
    runtime)`` returns the assembled model."""
    _REGISTRY[name] = (config_cls, builder)


def architectures():
    return sorted(_REGISTRY)


def lookup_architecture(name: str):
    try:
        return _REGISTRY[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}' (known: {', '.join(architectures()) or 'none'})"
        ) from None


def architecture_of(d: Dict[str, Any]) -> str:
    archs = d.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list holding the architecture's name")
    return archs[0]


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    config_cls, _ = lookup_architecture(architecture_of(d))
    cfg = config_cls.from_dict(d)
    cfg.validate()
    return cfg


def load_config(folder) -> ModelConfig:
    path = Path(folder) / "config.json"
    try:
        d = json.loads(path.read_text())
    except FileNotFoundError:
        raise ConfigError(f"{path}: no config.json in the model folder") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    cfg = config_from_dict(d)
    # a folder's generation_config.json may name more end tokens than config.json (chat models end a
    # turn with another id than the text's end): a reply stops at any of them
    ids = generation_eos_ids(folder)
    if ids and hasattr(cfg, "eos_token_ids"):
        cfg.eos_token_ids = list(dict.fromkeys(list(cfg.eos_token_ids) + ids))
    return cfg


def generation_eos_ids(folder) -> list:
    """``eos_token_id`` of the folder's generation_config.json (an id or a list of ids); none when
    the file is absent."""
    path = Path(folder) / "generation_config.json"
    if not path.exists():
        return []
    try:
        g = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not JSON: {e}") from None
    eos = g.get("eos_token_id") if isinstance(g, dict) else None
    if eos is None:
        return []
    try:
        return [int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)]
    except (TypeError, ValueError):
        raise ConfigError(f"{path}: 'eos_token_id' must be an id or a list of ids") from None
