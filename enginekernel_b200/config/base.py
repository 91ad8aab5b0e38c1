"""Typed model configurations read from a checkpoint's ``config.json``.

A configuration class declares its fields as dataclass fields whose metadata
names the ``config.json`` key they come from.  Reading is strict about types and
about keys the architecture needs; it never substitutes a size that the file
does not give.  The reference reads the same file into an untyped attribute bag
(engine/ek_model.py:26-42); the keys and defaults of each architecture are listed
in its own module.
"""

from __future__ import annotations

import dataclasses
import json
import os
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A ``config.json`` is missing a key, has a wrong type or is inconsistent."""


_REQUIRED = object()


def key(name: str, default: Any = _REQUIRED, doc: str = ""):
    """A dataclass field filled from ``config.json[name]``.

    Without ``default`` the key is required.
    """
    meta = {"json_key": name, "doc": doc, "required": default is _REQUIRED}
    if default is _REQUIRED:
        return dataclasses.field(metadata=meta)
    return dataclasses.field(default=default, metadata=meta)


@dataclasses.dataclass(frozen=True)
class ModelConfig:
    """Base of all architecture configurations."""

    #: value of ``config.json["architectures"][0]`` this class answers to
    architecture: ClassVar[str] = ""

    # -- construction -----------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "ModelConfig":
        if not isinstance(raw, dict):
            raise ConfigError(f"config must be a JSON object, got {type(raw).__name__}")
        values = {}
        for f in dataclasses.fields(cls):
            name = f.metadata.get("json_key")
            if name is None:
                continue
            if name in raw and raw[name] is not None:
                values[f.name] = _coerce(name, raw[name], f.type)
            elif f.metadata["required"]:
                fallback = cls._derive_missing(f.name, raw)
                if fallback is None:
                    raise ConfigError(f"config.json lacks the required key {name!r} "
                                      f"for {cls.architecture or cls.__name__}")
                values[f.name] = fallback
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path: str) -> "ModelConfig":
        """``path`` is a model folder or the ``config.json`` itself."""
        return cls.from_dict(read_config_json(path))

    @classmethod
    def _derive_missing(cls, field_name: str, raw: dict):
        """Value of a required field that the file may leave out (None: it may not)."""
        return None

    # -- checks and output --------------------------------------------------
    def validate(self) -> None:
        """Raise :class:`ConfigError` on sizes that cannot form a model."""

    def to_dict(self) -> dict:
        """The ``config.json`` content that reads back to this configuration."""
        out = {"architectures": [self.architecture]}
        for f in dataclasses.fields(self):
            name = f.metadata.get("json_key")
            if name is not None:
                out[name] = getattr(self, f.name)
        return out

    def replace(self, **changes) -> "ModelConfig":
        cfg = dataclasses.replace(self, **changes)
        cfg.validate()
        return cfg


def read_config_json(path: str) -> dict:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.exists(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        try:
            return json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path} is not valid JSON: {e}") from None


def _coerce(name: str, value: Any, annotation: Any):
    kind = annotation if isinstance(annotation, str) else getattr(annotation, "__name__", str(annotation))
    if kind == "int":
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ConfigError(f"config key {name!r} must be an integer, got {value!r}")
        return int(value)
    if kind == "float":
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key {name!r} must be a number, got {value!r}")
        return float(value)
    if kind == "bool":
        if not isinstance(value, bool):
            raise ConfigError(f"config key {name!r} must be true or false, got {value!r}")
        return value
    if kind == "str":
        if not isinstance(value, str):
            raise ConfigError(f"config key {name!r} must be a string, got {value!r}")
        return value
    return value
