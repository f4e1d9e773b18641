"""Typed access to the keys of a config.json dictionary.

Every architecture's configuration class reads its keys through a
``KeyReader``: a wrong type, a missing required key or a value outside its
range becomes one ``ConfigError`` that names the key.  The reference never
reads config.json (it infers sizes from tensor shapes and GGUF metadata,
src/engine/tq_model.c:949-1081, 2867-2905); the typed reader is this
library's own.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot describe a model: the message names the key."""


_MISSING = object()


class KeyReader:
    def __init__(self, raw: Dict[str, Any], where: str = "config.json"):
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: top level must be a JSON object")
        self.raw = raw
        self.where = where
        self.seen: set = set()

    def _get(self, key: str, default: Any) -> Any:
        self.seen.add(key)
        if key not in self.raw or self.raw[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.raw[key]

    def has(self, key: str) -> bool:
        return key in self.raw and self.raw[key] is not None

    def integer(self, key: str, default: Any = _MISSING, minimum: Optional[int] = None) -> int:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return int(v)

    def real(self, key: str, default: Any = _MISSING, positive: bool = False) -> float:
        v = self._get(key, default)
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def int_list(self, key: str, default: Any = _MISSING) -> List[int]:
        v = self._get(key, default)
        if not isinstance(v, (list, tuple)) or any(isinstance(i, bool) or not isinstance(i, int) for i in v):
            raise ConfigError(f"{self.where}: key '{key}' must be a list of integers, got {v!r}")
        return [int(i) for i in v]

    def token_ids(self, key: str) -> List[int]:
        """A key that holds one token id or a list of them (eos_token_id); [] if absent."""
        self.seen.add(key)
        v = self.raw.get(key)
        if v is None:
            return []
        if isinstance(v, int) and not isinstance(v, bool):
            return [int(v)]
        if isinstance(v, (list, tuple)) and all(isinstance(i, int) and not isinstance(i, bool) for i in v):
            return [int(i) for i in v]
        raise ConfigError(f"{self.where}: key '{key}' must be a token id or a list of them, got {v!r}")


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in model folder '{folder}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            raw = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path}: top level must be a JSON object")
    return raw
