"""One registry from an architecture's name to its configuration class and plan builder.

``config.json`` names its architecture in ``architectures[0]``; a GGUF file
names it in ``general.architecture``.  Both spellings are registered for the
same entry, so the model class is chosen the same way everywhere.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .plan import ModelPlan


class ConfigError(ValueError):
    """A configuration that is missing a key, holds a bad value or names an unknown architecture."""


@dataclass(frozen=True)
class Architecture:
    name: str
    from_dict: Callable[[Mapping[str, Any]], Any]      # config.json dict -> typed configuration
    build_plan: Callable[[Any], ModelPlan]             # typed configuration -> plan
    aliases: tuple[str, ...] = ()
    # GGUF support, if the architecture has it: metadata (and tensor shapes) -> config.json
    # dictionary, and the GGUF name of a checkpoint tensor name
    config_from_gguf: Any = None
    gguf_tensor_name: Any = None


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> None:
    for key in (arch.name, *arch.aliases):
        _ARCHITECTURES[key] = arch


def known_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture {name!r}; known: {', '.join(known_architectures())}") from None


def architecture_of(cfg: Mapping[str, Any]) -> Architecture:
    archs = cfg.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return get_architecture(archs[0])


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as fh:
            cfg = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"{path}: no such file") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path}: not valid JSON ({exc})") from None
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return cfg


def load_config(model_dir: str):
    """Read ``config.json`` and return ``(architecture, typed configuration)``."""
    cfg = read_config_json(model_dir)
    arch = architecture_of(cfg)
    return arch, arch.from_dict(cfg)
