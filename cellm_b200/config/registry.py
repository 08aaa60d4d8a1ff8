"""One registry from an architecture's name to its configuration class and
plan builder (tools/infer/src/main.rs:186-201 dispatches on `model_type` the
same way, and lists what it found when nothing matches)."""
from __future__ import annotations

import json
import os
from typing import Callable

from .errors import ConfigError
from .plan import ModelPlan

_ARCHITECTURES: dict[str, tuple[type, Callable[[object], ModelPlan]]] = {}
_MODEL_TYPES: dict[str, str] = {}


def register_architecture(name: str, config_cls: type, build_plan, model_types=()) -> None:
    """`name` is what config.json lists under `architectures`; `model_types`
    are accepted values of `model_type` when `architectures` is absent."""
    _ARCHITECTURES[name] = (config_cls, build_plan)
    for t in model_types:
        _MODEL_TYPES[t] = name


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def _effective_model_type(d: dict):
    # tools/infer/src/main.rs:1062-1071 prefers the text config's model_type.
    tc = d.get("text_config")
    if isinstance(tc, dict) and tc.get("model_type"):
        return tc["model_type"]
    return d.get("model_type")


def resolve_architecture(d: dict) -> str:
    archs = d.get("architectures") or []
    for a in archs:
        if a in _ARCHITECTURES:
            return a
    mt = _effective_model_type(d)
    if mt in _MODEL_TYPES:
        return _MODEL_TYPES[mt]
    raise ConfigError(
        f"unsupported model: architectures={archs!r} model_type={mt!r}; "
        f"registered architectures: {registered_architectures()}, "
        f"model types: {sorted(_MODEL_TYPES)}")


def config_from_dict(d: dict):
    """(typed configuration, plan) for a config.json dictionary."""
    name = resolve_architecture(d)
    config_cls, build_plan = _ARCHITECTURES[name]
    cfg = config_cls.from_dict(d)
    plan = build_plan(cfg)
    plan.validate()
    return cfg, plan


def load_config(folder: str):
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in {folder!r}")
    with open(path) as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return config_from_dict(d)
