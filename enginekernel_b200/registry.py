"""Registries: architecture name -> (configuration class, model builder), and
part kind -> part class.

The reference hard-wires one model class (engine/engine.py:82,196).  Here the
name in ``config.json["architectures"][0]`` selects the configuration class and a
builder that turns the configuration into a :class:`~enginekernel_b200.parts.spec.ModelSpec`
(pure data: which parts, in which order).  Parts (mixers, feed-forwards, norms,
position encodings, block arrangements) are registered by role and kind, so a new
part or a whole architecture is added by registering it - from outside the
package too - without editing any file here.
"""

from __future__ import annotations

from typing import Callable, Dict, Tuple, Type

from .config.base import ConfigError, ModelConfig, read_config_json

_ARCHITECTURES: Dict[str, Tuple[Type[ModelConfig], Callable]] = {}
_PARTS: Dict[Tuple[str, str], type] = {}

PART_ROLES = ("mixer", "feed_forward", "norm", "position", "block")


class RegistryError(KeyError):
    def __str__(self):  # KeyError quotes its message; keep it readable
        return self.args[0] if self.args else ""


# -- architectures ------------------------------------------------------------
def register_architecture(name: str, config_cls: Type[ModelConfig], builder: Callable,
                          *, replace: bool = False) -> None:
    """``builder(config) -> ModelSpec``."""
    if name in _ARCHITECTURES and not replace:
        raise RegistryError(f"architecture {name!r} is already registered")
    _ARCHITECTURES[name] = (config_cls, builder)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures():
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def lookup_architecture(name: str):
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise RegistryError(f"unknown architecture {name!r}; registered: "
                            f"{', '.join(sorted(_ARCHITECTURES)) or 'none'}") from None


def architecture_of(raw_config: dict) -> str:
    names = raw_config.get("architectures")
    if not (isinstance(names, list) and names and isinstance(names[0], str)):
        raise ConfigError('config.json needs "architectures": ["<name>"] to choose the model')
    return names[0]


def config_from_folder(path: str) -> ModelConfig:
    """Read ``config.json`` and build the typed configuration its architecture names."""
    raw = read_config_json(path)
    config_cls, _ = lookup_architecture(architecture_of(raw))
    return config_cls.from_dict(raw)


def model_spec_for(config: ModelConfig):
    _, builder = lookup_architecture(config.architecture)
    return builder(config)


# -- parts ----------------------------------------------------------------------
def register_part(role: str, kind: str, cls: type = None, *, replace: bool = False):
    """Register ``cls`` as the part ``kind`` of ``role``; usable as a decorator."""
    if role not in PART_ROLES:
        raise RegistryError(f"unknown part role {role!r}; roles: {', '.join(PART_ROLES)}")

    def put(c):
        if (role, kind) in _PARTS and not replace:
            raise RegistryError(f"{role} {kind!r} is already registered")
        _PARTS[(role, kind)] = c
        return c

    return put(cls) if cls is not None else put


def unregister_part(role: str, kind: str) -> None:
    _PARTS.pop((role, kind), None)


def lookup_part(role: str, kind: str) -> type:
    _ensure_builtin()
    try:
        return _PARTS[(role, kind)]
    except KeyError:
        known = sorted(k for r, k in _PARTS if r == role)
        raise RegistryError(f"unknown {role} kind {kind!r}; registered: "
                            f"{', '.join(known) or 'none'}") from None


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from . import models  # noqa: F401  (registers architectures)
        from . import parts  # noqa: F401   (registers parts)
