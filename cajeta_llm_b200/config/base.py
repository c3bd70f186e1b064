"""Typed model configuration and the architecture registry.

A configuration class reads the architecture's own ``config.json`` keys into typed
fields and validates them.  No size and no constant that ``config.json`` gives is
repeated anywhere else in the package: every part receives its sizes as parameters
taken from the configuration object.

The reference keeps one ``ModelConfig`` with every family's fields
(model/ModelConfig.cajeta:25-108), names file and key for a missing required key
(model/ModelConfig.cajeta:604-611) and lists the supported architectures when the
name is unknown (model/ModelConfig.cajeta:358-364).  Here each architecture owns a
small dataclass and registers it by its ``architectures[0]`` string.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, fields
from typing import Any, Callable, Dict, Type


class ConfigError(ValueError):
    """A ``config.json`` that cannot be used: names the key and the reason."""


_MISSING = object()


class ConfigReader:
    """Typed access to the keys of one ``config.json`` with errors that name the key."""

    def __init__(self, raw: Dict[str, Any], source: str = "config.json"):
        self.raw = raw
        self.source = source

    def _get(self, key: str, default: Any = _MISSING) -> Any:
        if key in self.raw and self.raw[key] is not None:
            return self.raw[key]
        if default is _MISSING:
            raise ConfigError(f"{self.source}: required key '{key}' is missing")
        return default

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None) -> int:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.source}: key '{key}' must be an integer, found {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.source}: key '{key}' must be >= {minimum}, found {v}")
        return int(v)

    def optional_integer(self, key: str) -> int | None:
        if self.raw.get(key) is None:
            return None
        return self.integer(key)

    def number(self, key: str, default: Any = _MISSING) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.source}: key '{key}' must be a number, found {v!r}")
        return float(v)

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.source}: key '{key}' must be true or false, found {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.source}: key '{key}' must be a string, found {v!r}")
        return v

    def integer_list(self, key: str, default: Any = _MISSING) -> tuple:
        v = self._get(key, default)
        if isinstance(v, int) and not isinstance(v, bool):
            v = [v]
        if not isinstance(v, (list, tuple)) or any(isinstance(x, bool) or not isinstance(x, int) for x in v):
            raise ConfigError(f"{self.source}: key '{key}' must be a list of integers, found {v!r}")
        return tuple(int(x) for x in v)


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    Subclasses add their fields, implement :meth:`from_reader` (config.json keys to
    fields) and :meth:`to_json_dict` (fields back to config.json keys, used by the
    random-weights mode to write a model folder).
    """

    architecture: str

    @classmethod
    def from_reader(cls, r: ConfigReader) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_json_dict(self) -> Dict[str, Any]:  # pragma: no cover - abstract
        raise NotImplementedError

    def replace(self, **changes: Any) -> "ModelConfig":
        values = {f.name: getattr(self, f.name) for f in fields(self)}
        values.update(changes)
        return type(self)(**values)


@dataclass
class Architecture:
    """What the registry holds for one ``architectures[0]`` name.

    ``config_class`` parses config.json; ``build_plan`` turns a configuration into a
    :class:`cajeta_llm_b200.parts.plan.ModelPlan` (layer specs, run order, tensor names).
    """

    name: str
    config_class: Type[ModelConfig]
    build_plan: Callable[[ModelConfig], Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Type[ModelConfig],
                          build_plan: Callable[[ModelConfig], Any], replace: bool = False) -> Architecture:
    """Add an architecture to the one registry (name -> configuration class + plan builder)."""
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    arch = Architecture(name=name, config_class=config_class, build_plan=build_plan)
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> tuple:
    return tuple(sorted(_ARCHITECTURES))


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(
            f"unsupported architecture '{name}'; registered: {', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def parse_config_dict(raw: Dict[str, Any], source: str = "config.json") -> ModelConfig:
    """Choose the configuration class by ``architectures[0]`` and parse the keys."""
    archs = raw.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{source}: required key 'architectures' is missing or is not a list of names")
    arch = get_architecture(archs[0])
    return arch.config_class.from_reader(ConfigReader(raw, source))


def load_config(model_dir: str) -> ModelConfig:
    """Read ``<model_dir>/config.json``."""
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return parse_config_dict(raw, path)
