"""One registry from an architecture's name to its configuration class and model builder.

The reference admits a model by looking its architecture string up in an
allow-list and refuses everything else with a message that names the string
(`model_supported_archs`, src/model.c:751-763; refusal src/model.c:1384-1418).
This registry keeps that shape: ``resolve`` returns the entry or raises an
error listing the names it knows.  An entry is data: the class that types
config.json and a function that turns a configuration into a model
description (see ``engine.model``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Optional

from .base import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict], Any]
    build_plan: Callable[[Any], Any]      # configuration -> engine.model.ModelPlan
    # run-time overrides of the configuration that the entry points offer (the reference's --rope-base and
    # --rope-scale, src/model.c:282, 324-326): (configuration, rope_base=..., rope_scale=...) -> configuration, or
    # None when the architecture has nothing of the kind
    override: Optional[Callable[..., Any]] = None


_ARCHITECTURES: Dict[str, Architecture] = {}


class UnknownArchitecture(ConfigError):
    pass


def register_architecture(name: str, config_from_dict, build_plan, *, override=None, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_plan, override)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def resolve(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitecture(
            f"architecture '{name}' is not supported; known: {', '.join(known_architectures()) or '(none)'}"
        ) from None


def load_config(model_dir: str):
    """Read config.json of a model folder; the class is chosen by `architectures[0]`.

    Returns (architecture entry, typed configuration).
    """
    d = read_config_json(model_dir)
    archs = d.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError("config.json: 'architectures' must be a list holding one name")
    arch = resolve(archs[0])
    return arch, arch.config_from_dict(d)
