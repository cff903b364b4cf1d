"""Registries: architecture name -> model builder, and part kind -> part class.

The architecture rule is the reference's (src/models/layer_key_prefix.cpp:24-28,
92-105): lower-case ``architectures[0]`` and ``model_type``; an entry matches if
its key occurs in the architecture string or equals the model type; no match
raises ``ValueError`` naming both strings.

Parts are looked up by ``PartSpec.kind`` in one of five tables (mixer,
feed_forward, norm, position, and head for embedding / lm_head).  A test or a
user registers another kind with ``register_part`` without touching this
package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from .config.spec import ModelSpec


@dataclass(frozen=True)
class Architecture:
    key: str                                  # matched against architectures[0] / model_type, lower case
    config_from_dict: Callable[[dict], object]  # typed configuration from the config.json dict
    build_spec: Callable[[object], ModelSpec]   # typed configuration -> ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}
_PARTS: Dict[str, Dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "head": {}}


def register_architecture(key: str, config_from_dict, build_spec) -> None:
    _ARCHITECTURES[key.lower()] = Architecture(key.lower(), config_from_dict, build_spec)


def resolve_architecture(config_dict: dict) -> Architecture:
    arch = ""
    archs = config_dict.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        arch = archs[0]
    model_type = str(config_dict.get("model_type", ""))
    for key, entry in _ARCHITECTURES.items():
        if key in arch.lower() or model_type.lower() == key:
            return entry
    raise ValueError("Unsupported model architecture/model_type: "
                     f"architecture='{arch}', model_type='{model_type}'")


def model_spec_from_config(config_dict: dict) -> ModelSpec:
    entry = resolve_architecture(config_dict)
    return entry.build_spec(entry.config_from_dict(config_dict))


def register_part(role: str, kind: str, cls: type) -> None:
    if role not in _PARTS:
        raise KeyError(f"unknown part role {role!r}; roles are {sorted(_PARTS)}")
    _PARTS[role][kind] = cls


def part_class(role: str, kind: str) -> type:
    try:
        return _PARTS[role][kind]
    except KeyError:
        raise KeyError(f"no {role} part of kind {kind!r} is registered "
                       f"(known: {sorted(_PARTS.get(role, {}))})") from None
