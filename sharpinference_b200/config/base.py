"""Typed reading of a model folder's ``config.json``.

The reference fills one typed record from model metadata with required keys that
throw and optional keys that default (src/SharpInference.Engine/DSparkConfig.cs:41-89,
src/SharpInference.Core/ModelGraph.cs:492-543).  ``ConfigReader`` is the same idea for
``config.json``: every access names the key, the wanted type and, for optional keys,
the default; all problems of one file are reported together.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Optional, Sequence


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


_MISSING = object()


class ConfigReader:
    """Reads typed values out of one JSON object and collects every problem.

    ``finish()`` raises one ``ConfigError`` that lists all of them, so a user fixes a
    config.json in one pass instead of one key at a time.
    """

    def __init__(self, obj: dict, where: str = "config.json"):
        if not isinstance(obj, dict):
            raise ConfigError(f"{where}: expected a JSON object, found {type(obj).__name__}")
        self._obj = obj
        self._where = where
        self._problems: list[str] = []

    # -- scalar access -----------------------------------------------------------------
    def _get(self, key: str, kind: str, conv: Callable[[Any], Any], default: Any) -> Any:
        value = self._obj.get(key, _MISSING)
        if value is _MISSING or value is None:
            if default is _MISSING:
                self._problems.append(f"missing required key '{key}' ({kind})")
                return None
            return default
        try:
            return conv(value)
        except (TypeError, ValueError) as exc:
            self._problems.append(f"key '{key}': expected {kind}, found {value!r} ({exc})")
            return None if default is _MISSING else default

    @staticmethod
    def _as_int(value: Any) -> int:
        if isinstance(value, bool):
            raise TypeError("a boolean is not an integer")
        if isinstance(value, float):
            if value != int(value):
                raise ValueError("not a whole number")
            return int(value)
        if not isinstance(value, int):
            raise TypeError(f"{type(value).__name__}")
        return value

    @staticmethod
    def _as_float(value: Any) -> float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise TypeError(f"{type(value).__name__}")
        return float(value)

    @staticmethod
    def _as_bool(value: Any) -> bool:
        if not isinstance(value, bool):
            raise TypeError(f"{type(value).__name__}")
        return value

    @staticmethod
    def _as_str(value: Any) -> str:
        if not isinstance(value, str):
            raise TypeError(f"{type(value).__name__}")
        return value

    def int(self, key: str, default: Any = _MISSING) -> int:
        return self._get(key, "integer", self._as_int, default)

    def float(self, key: str, default: Any = _MISSING) -> float:
        return self._get(key, "number", self._as_float, default)

    def bool(self, key: str, default: Any = _MISSING) -> bool:
        return self._get(key, "boolean", self._as_bool, default)

    @staticmethod
    def _as_switch(value: Any) -> bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, int) and value >= 0:
            return value != 0
        raise TypeError(f"{type(value).__name__}")

    def switch(self, key: str, default: Any = _MISSING) -> bool:
        """A boolean that some files write as a non-negative integer (non-zero = on)."""
        return self._get(key, "boolean or non-negative integer", self._as_switch, default)

    def str(self, key: str, default: Any = _MISSING) -> str:
        return self._get(key, "string", self._as_str, default)

    def int_list(self, key: str, default: Any = _MISSING) -> Optional[list]:
        def conv(value: Any) -> list:
            if not isinstance(value, (list, tuple)):
                raise TypeError(f"{type(value).__name__}")
            return [self._as_int(v) for v in value]

        return self._get(key, "list of integers", conv, default)

    def object(self, key: str, default: Any = _MISSING) -> Optional[dict]:
        def conv(value: Any) -> dict:
            if not isinstance(value, dict):
                raise TypeError(f"{type(value).__name__}")
            return value

        return self._get(key, "object", conv, default)

    def has(self, key: str) -> bool:
        return self._obj.get(key, None) is not None

    # -- problems ----------------------------------------------------------------------
    def problem(self, text: str) -> None:
        self._problems.append(text)

    def require(self, condition: bool, text: str) -> None:
        if not condition:
            self._problems.append(text)

    @property
    def ok(self) -> bool:
        return not self._problems

    def finish(self) -> None:
        if self._problems:
            lines = "\n  - ".join(self._problems)
            raise ConfigError(f"{self._where}: {len(self._problems)} problem(s):\n  - {lines}")


def read_config_json(model_dir: str) -> dict:
    """Parse ``<model_dir>/config.json`` (or a path to the JSON file itself)."""
    path = model_dir if model_dir.endswith(".json") else os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no such file (a model folder holds config.json and model.safetensors)")
    with open(path, "r", encoding="utf-8") as fh:
        try:
            obj = json.load(fh)
        except json.JSONDecodeError as exc:
            raise ConfigError(f"{path}: not valid JSON: {exc}") from None
    if not isinstance(obj, dict):
        raise ConfigError(f"{path}: expected a JSON object at the top level")
    return obj


def architecture_name(obj: dict, where: str = "config.json") -> str:
    """The name under which the model class is registered: ``architectures[0]``."""
    archs = obj.get("architectures")
    if isinstance(archs, Sequence) and not isinstance(archs, str) and len(archs) >= 1 and isinstance(archs[0], str):
        return archs[0]
    raise ConfigError(f"{where}: key 'architectures' must be a non-empty list of names, found {archs!r}")
