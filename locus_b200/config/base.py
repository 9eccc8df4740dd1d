"""Typed model configuration and the architecture registry.

A model folder's ``config.json`` names its architecture in ``architectures[0]``.
The registry maps that name to an :class:`ArchEntry`: how to parse the typed
configuration and how to build the model from it.  Lookup of an unknown name
fails with an error that lists the supported names, in the manner of the
reference's ``find_arch`` (src/locus/model/arch.cpp:870-877) and its
unsupported-architecture message (src/locus/model/llama.cpp:168-180).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List


class ConfigError(ValueError):
    """A configuration that cannot be built: missing key, bad value, bad relation."""


@dataclass(frozen=True)
class ArchEntry:
    """One supported architecture.

    ``parse_config`` turns the raw ``config.json`` dictionary into the typed
    configuration; ``build_model`` turns that configuration into a
    :class:`locus_b200.models.plan.ModelPlan` (parts chosen layer by layer,
    the run order, the tensor names).  ``description`` is what ``--archs`` prints.
    """

    name: str
    description: str
    parse_config: Callable[[Dict[str, Any]], Any]
    build_plan: Callable[[Any], Any]


_ARCHS: Dict[str, ArchEntry] = {}


def register_arch(entry: ArchEntry) -> None:
    _ARCHS[entry.name] = entry


def archs() -> List[ArchEntry]:
    """All registered architectures in registration order."""
    return list(_ARCHS.values())


def find_arch(name: str) -> ArchEntry:
    try:
        return _ARCHS[name]
    except KeyError:
        supported = ", ".join(sorted(_ARCHS)) or "(none)"
        raise ConfigError(
            f"unsupported architecture: {name!r} (supported: {supported})"
        ) from None


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder: {model_dir}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json is not a JSON object: {path}")
    return raw


def arch_name_of(raw: Dict[str, Any]) -> str:
    names = raw.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("config.json: missing key: architectures")
    return names[0]


def load_config(model_dir: str):
    """(ArchEntry, typed configuration) of a model folder."""
    raw = read_config_json(model_dir)
    entry = find_arch(arch_name_of(raw))
    return entry, entry.parse_config(raw)


# ---------------------------------------------------------------------------
# helpers for typed parsing


_MISSING = object()


def take(raw: Dict[str, Any], key: str, kind, default=_MISSING):
    """``raw[key]`` as ``kind`` (int, float, bool, list); error names the key."""
    if key not in raw or raw[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: missing key: {key}")
        return default
    v = raw[key]
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: {key} must be true or false, got {v!r}")
        return v
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                return int(v)
            raise ConfigError(f"config.json: {key} must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {key} must be a number, got {v!r}")
        return float(v)
    if kind is list:
        if not isinstance(v, list):
            raise ConfigError(f"config.json: {key} must be a list, got {v!r}")
        return list(v)
    raise TypeError(kind)
