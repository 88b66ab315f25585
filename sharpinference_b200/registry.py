"""One registry from an architecture's name to its configuration class and model builder.

The reference switches on the model's architecture string in many places
(src/SharpInference.Core/ModelGraph.cs:262, :294, :308-328) and picks the forward-pass
class in the command line (src/SharpInference.Cli/RunCommand.cs:618-633).  Here the name
in ``config.json`` (``architectures[0]``) selects everything through this one table, and
nothing else in the framework knows a model's name.

An architecture supplies two things:

``config_cls``
    a class with ``from_dict(obj, where) -> config`` and ``to_dict() -> dict``;
``build(config, weights, options) -> DecoderModel``
    a function that puts the model together from parts and asks ``weights`` (a
    :class:`sharpinference_b200.weights.WeightSource`) for every tensor by its name in the
    file.  The same function run against a declaring source yields the list of tensors a
    model folder must hold, which is what the random-weights writer uses.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from .config.base import ConfigError, architecture_name


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: Any
    build: Callable[..., Any]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: Any, build: Callable[..., Any], *, aliases=()) -> Architecture:
    """Add (or replace) an architecture.  ``aliases`` are further names that select it."""
    arch = Architecture(name=name, config_cls=config_cls, build=build)
    for key in (name, *aliases):
        _ARCHITECTURES[key] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures() -> list:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(
            f"unknown architecture '{name}'; registered: {', '.join(sorted(_ARCHITECTURES)) or '(none)'}"
        ) from None


def resolve(config_obj: dict, where: str = "config.json"):
    """``(architecture, typed config)`` for a parsed config.json."""
    arch = get_architecture(architecture_name(config_obj, where))
    return arch, arch.config_cls.from_dict(config_obj, where)


_builtin_loaded = False


def _ensure_builtin() -> None:
    global _builtin_loaded
    if not _builtin_loaded:
        _builtin_loaded = True
        from .models import llama4  # noqa: F401  (registers itself)
