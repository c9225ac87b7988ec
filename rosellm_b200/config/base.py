"""Typed model configurations and the registry from architecture name to model.

A model folder holds ``config.json``; its ``architectures[0]`` (or, failing
that, ``model_type``) names the architecture.  The registry maps that name to
a configuration class, which parses the architecture's own ``config.json``
keys, and to a builder, which turns a parsed configuration into a
``ModelSpec`` (see ``rosellm_b200.parts.spec``).  Nothing else in the package
knows an architecture's name.

The reference picks its model with an ``if model_type == "gpt2" ... elif``
chain (rosellm/roseinfer/mp.py:663-697) and refuses anything but GPT-2 in
rosellm/rosetrainer/hf_gpt2.py:99-102; here the same decision is one
dictionary so that another architecture is one ``register_architecture`` call.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` that is missing a key, or holds a value no part supports."""


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's typed configuration."""

    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict[str, Any]:
        """The ``config.json`` content that ``from_dict`` parses back to ``self``."""
        raise NotImplementedError

    def flat(self) -> dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self)}


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type[ModelConfig]
    build_spec: Callable[[ModelConfig], Any]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(
    name: str,
    config_cls: type[ModelConfig],
    build_spec: Callable[[ModelConfig], Any],
    model_types: tuple[str, ...] = (),
    *,
    replace: bool = False,
) -> None:
    """Make ``name`` (a value of ``config.json``'s ``architectures``) loadable.

    ``build_spec(config)`` returns the ``ModelSpec`` of parts, layer by layer.
    ``model_types`` are ``model_type`` values accepted when ``architectures``
    is absent.
    """
    if name in _ARCHITECTURES and not replace:
        raise ConfigError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec, tuple(model_types))


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def resolve_architecture(raw: dict[str, Any]) -> Architecture:
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for name in names:
        if name in _ARCHITECTURES:
            return _ARCHITECTURES[name]
    model_type = raw.get("model_type")
    if not names and model_type is not None:
        for arch in _ARCHITECTURES.values():
            if model_type in arch.model_types:
                return arch
    raise ConfigError(
        f"unknown architecture: architectures={names!r} model_type={model_type!r}; "
        f"registered: {registered_architectures()}"
    )


def parse_config(raw: dict[str, Any]) -> ModelConfig:
    return resolve_architecture(raw).config_cls.from_dict(raw)


def read_config_json(model_dir: str) -> dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json in model folder {model_dir!r}")
    with open(path, "r", encoding="utf-8") as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return raw


def load_config(model_dir: str) -> ModelConfig:
    return parse_config(read_config_json(model_dir))


def require(raw: dict[str, Any], key: str, kind: type, *alternatives: str) -> Any:
    """``raw[key]`` (or the first alternative present) checked to be ``kind``."""
    for k in (key, *alternatives):
        if k in raw and raw[k] is not None:
            value = raw[k]
            if kind is float and isinstance(value, int) and not isinstance(value, bool):
                value = float(value)
            if not isinstance(value, kind) or isinstance(value, bool) and kind is not bool:
                raise ConfigError(f"config.json: {k!r} must be {kind.__name__}, got {value!r}")
            return value
    names = " or ".join(repr(k) for k in (key, *alternatives))
    raise ConfigError(f"config.json: missing required key {names}")


def optional(raw: dict[str, Any], key: str, kind: type, default: Any) -> Any:
    if key not in raw or raw[key] is None:
        return default
    return require(raw, key, kind)
