"""Typed reading of a model folder's ``config.json``.

The reference passes an untyped ``AutoConfig`` object around and probes it with
``hasattr`` (cpmcu/llm.py:46, 62-69).  Here every architecture declares a typed
configuration; the helpers below turn JSON values into typed fields and collect
every problem of a file into one error.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, List, Optional, Sequence


class ConfigError(ValueError):
    """A ``config.json`` that is missing keys, has wrong types or impossible sizes."""


_MISSING = object()


class FieldReader:
    """Reads keys of one JSON object, remembering which were used and what went wrong."""

    def __init__(self, data: Dict[str, Any], where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object, got {type(data).__name__}")
        self.data = data
        self.where = where
        self.problems: List[str] = []
        self.used: set = set()

    def _get(self, key: str, default: Any = _MISSING) -> Any:
        self.used.add(key)
        if key in self.data and self.data[key] is not None:
            return self.data[key]
        if default is _MISSING:
            self.problems.append(f"{self.where}: required key '{key}' is missing")
            return None
        return default

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> Optional[int]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                v = int(v)
            else:
                self.problems.append(f"{self.where}: '{key}' must be an integer, got {v!r}")
                return None
        if minimum is not None and v < minimum:
            self.problems.append(f"{self.where}: '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False) -> Optional[float]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            self.problems.append(f"{self.where}: '{key}' must be a number, got {v!r}")
            return None
        v = float(v)
        if positive and not v > 0:
            self.problems.append(f"{self.where}: '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> Optional[bool]:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, bool):
            self.problems.append(f"{self.where}: '{key}' must be true or false, got {v!r}")
            return None
        return v

    def string(self, key: str, default: Any = _MISSING, choices: Optional[Sequence[str]] = None) -> Optional[str]:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, str):
            self.problems.append(f"{self.where}: '{key}' must be a string, got {v!r}")
            return None
        if choices is not None and v not in choices:
            self.problems.append(f"{self.where}: '{key}' must be one of {list(choices)}, got {v!r}")
        return v

    def numbers(self, key: str, default: Any = _MISSING) -> Optional[List[float]]:
        v = self._get(key, default)
        if v is None:
            return None
        if not isinstance(v, (list, tuple)) or any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in v):
            self.problems.append(f"{self.where}: '{key}' must be a list of numbers")
            return None
        return [float(x) for x in v]

    def int_or_ints(self, key: str, default: Any = _MISSING) -> Optional[List[int]]:
        v = self._get(key, default)
        if v is None:
            return None
        if isinstance(v, int) and not isinstance(v, bool):
            return [v]
        if isinstance(v, (list, tuple)) and all(isinstance(x, int) and not isinstance(x, bool) for x in v):
            return [int(x) for x in v]
        self.problems.append(f"{self.where}: '{key}' must be an integer or a list of integers")
        return None

    def child(self, key: str) -> Optional["FieldReader"]:
        """A nested object, or None when the key is absent or null."""
        self.used.add(key)
        v = self.data.get(key)
        if v is None:
            return None
        if not isinstance(v, dict):
            self.problems.append(f"{self.where}: '{key}' must be an object or null")
            return None
        return FieldReader(v, f"{self.where}:{key}")

    def absorb(self, child: Optional["FieldReader"]) -> None:
        if child is not None:
            self.problems.extend(child.problems)

    def check(self, ok: bool, message: str) -> None:
        if not ok:
            self.problems.append(f"{self.where}: {message}")

    def finish(self) -> None:
        if self.problems:
            raise ConfigError("invalid configuration:\n  " + "\n  ".join(self.problems))


def read_config_json(model_dir_or_file: str) -> Dict[str, Any]:
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path, "r", encoding="utf-8") as f:
        try:
            data = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return data


def architecture_name(data: Dict[str, Any]) -> str:
    """The name a model folder asks for: ``architectures[0]`` of its config.json.

    The reference guesses from substrings of ``architectures[0]``/``model_type`` and
    from ``num_hidden_layers / num_key_value_heads`` (cpmcu/common/utils.py:33-64);
    here the name is taken as written.
    """
    arch = data.get("architectures")
    if isinstance(arch, (list, tuple)) and arch and isinstance(arch[0], str):
        return arch[0]
    if isinstance(arch, str):
        return arch
    raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
