"""Typed configurations and the one registry from an architecture's name to its model.

ember.cpp parses `config.json` into a struct with `json.value(key, default)` and takes
`architectures[0]` as the architecture (model_config.cpp:20-45); it looks for `config.json` in the
model folder (safetensors_loader.cpp:607-681).  Its closest thing to a registry is the set of
architectures it can build a graph for, named in the error when one is missing
(graph_ir.cpp:523-527, 551-554).  Here the registry is explicit: a name maps to a configuration
class and to a function that turns a configuration into a `ModelSpec` (data, see parts/spec.py).
"""
from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, Callable, ClassVar


class ConfigError(ValueError):
    """A configuration that cannot be used; the message names the key."""


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.  Subclasses list the architecture's own
    config.json keys as fields; `from_dict` reads them and `validate` refuses what the parts
    cannot run."""

    architecture: ClassVar[str] = ""
    # alias -> canonical key, per subclass
    aliases: ClassVar[dict[str, str]] = {}

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "ModelConfig":
        known = {f.name: f for f in dataclasses.fields(cls)}
        values: dict[str, Any] = {}
        for alias, key in cls.aliases.items():
            if alias in d and key not in d:
                values[key] = d[alias]
        for key, f in known.items():
            if key in d and d[key] is not None:
                values[key] = d[key]
        missing = [k for k, f in known.items()
                   if k not in values and f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING]
        if missing:
            raise ConfigError(f"{cls.__name__}: config.json has no {', '.join(repr(m) for m in missing)}")
        for key, val in list(values.items()):
            want = known[key].type
            values[key] = _coerce(cls.__name__, key, val, want)
        cfg = cls(**values)
        cfg.validate()
        return cfg

    def validate(self) -> None:  # pragma: no cover - overridden
        pass

    def check_dtype(self, dtype: str) -> None:
        """Refuses a configuration that the kernels of compute type `dtype` cannot run, naming the
        key; called before any weight is read.  The default refuses nothing."""

    def to_dict(self) -> dict[str, Any]:
        d = dataclasses.asdict(self)
        d["architectures"] = [self.architecture]
        return d


def _coerce(owner: str, key: str, val: Any, want: Any) -> Any:
    name = want if isinstance(want, str) else getattr(want, "__name__", str(want))
    name = name.replace(" ", "")
    try:
        if name.startswith("int"):
            if isinstance(val, bool) or (isinstance(val, float) and int(val) != val):
                raise TypeError
            return int(val)
        if name.startswith("float"):
            if isinstance(val, bool):
                raise TypeError
            return float(val)
        if name.startswith("bool"):
            if not isinstance(val, bool):
                raise TypeError
            return val
        if name.startswith("str"):
            if not isinstance(val, str):
                raise TypeError
            return val
    except (TypeError, ValueError):
        raise ConfigError(f"{owner}: key {key!r} has value {val!r}, expected {name}") from None
    return val


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build_spec: Callable[[ModelConfig], Any]


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build_spec: Callable[[ModelConfig], Any]) -> None:
    """Adds (or replaces) an architecture: `config_cls.from_dict` reads its config.json,
    `build_spec(config)` returns the ModelSpec that the engine builds and runs."""
    _ARCHITECTURES[name] = Architecture(name, config_cls, build_spec)


def architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"architecture {name!r} is not registered; registered: {', '.join(architectures()) or 'none'}")
    return _ARCHITECTURES[name]


def config_from_dict(d: dict[str, Any]) -> ModelConfig:
    arch = d.get("architectures")
    if not isinstance(arch, list) or not arch or not isinstance(arch[0], str):
        raise ConfigError("config.json has no 'architectures' list naming the model class")
    return get_architecture(arch[0]).config_cls.from_dict(d)


def load_config(folder: str) -> ModelConfig:
    """Reads `<folder>/config.json`; the class is chosen by `architectures[0]`."""
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        with open(path) as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level is not an object")
    return config_from_dict(d)
