"""Strictly typed access to a model folder's config.json.

The reference reads config.json into a flat key/value table whose getters stop the program when a
key holds another JSON type than the one asked for, and return "absent" for a missing key
(hf_config.h:59-79, hf_config.c:292-319).  `ConfigFields` keeps that contract, with exceptions in
place of exits, and also materialises arrays (the reference only types them, hf_config.h:9-17),
because the architecture name lives in `architectures[0]`.
"""
from __future__ import annotations

import json
import os
from typing import Any, List, Optional


class ConfigError(ValueError):
    """A config.json that cannot be used: missing key, wrong type, unsupported value."""


_ABSENT = object()


class ConfigFields:
    def __init__(self, table: dict, origin: str = "<dict>"):
        if not isinstance(table, dict):
            raise ConfigError(f"{origin}: the top level of config.json must be an object")
        self.table = table
        self.origin = origin

    @classmethod
    def from_file(cls, path: str) -> "ConfigFields":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        try:
            with open(path, "r", encoding="utf-8") as f:
                text = f.read()
        except OSError as e:
            raise ConfigError(f"could not open {path} ({e.strerror})") from e
        if not text.strip():
            raise ConfigError(f"{path} is empty")
        try:
            table = json.loads(text)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from e
        return cls(table, path)

    def has(self, key: str) -> bool:
        return key in self.table

    def is_null(self, key: str) -> bool:
        return key in self.table and self.table[key] is None

    def _get(self, key: str, default: Any, required: bool):
        v = self.table.get(key, _ABSENT)
        if v is _ABSENT or v is None:
            if required:
                raise ConfigError(f"{self.origin} missing '{key}'")
            return default, False
        return v, True

    def integer(self, key: str, default: Optional[int] = None, required: bool = False) -> Optional[int]:
        v, found = self._get(key, default, required)
        if not found:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.origin}: key '{key}' is not a number")
        if isinstance(v, float):
            if v != int(v):
                raise ConfigError(f"{self.origin}: key '{key}' = {v} is not an integer")
            v = int(v)
        return v

    def number(self, key: str, default: Optional[float] = None, required: bool = False) -> Optional[float]:
        v, found = self._get(key, default, required)
        if not found:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.origin}: key '{key}' is not a number")
        return float(v)

    def boolean(self, key: str, default: Optional[bool] = None, required: bool = False) -> Optional[bool]:
        v, found = self._get(key, default, required)
        if not found:
            return v
        if not isinstance(v, bool):
            raise ConfigError(f"{self.origin}: key '{key}' is not a bool")
        return v

    def string(self, key: str, default: Optional[str] = None, required: bool = False) -> Optional[str]:
        v, found = self._get(key, default, required)
        if not found:
            return v
        if not isinstance(v, str):
            raise ConfigError(f"{self.origin}: key '{key}' is not a string")
        return v

    def string_list(self, key: str) -> Optional[List[str]]:
        v, found = self._get(key, None, False)
        if not found:
            return None
        if not isinstance(v, list) or not all(isinstance(s, str) for s in v):
            raise ConfigError(f"{self.origin}: key '{key}' is not an array of strings")
        return list(v)

    def integer_or_list(self, key: str) -> List[int]:
        """A key such as eos_token_id, which is a number in some folders and an array in others."""
        v, found = self._get(key, None, False)
        if not found:
            return []
        if isinstance(v, list):
            if not all(isinstance(i, int) and not isinstance(i, bool) for i in v):
                raise ConfigError(f"{self.origin}: key '{key}' is not an array of integers")
            return list(v)
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"{self.origin}: key '{key}' is not a number")
        return [v]

    def mapping(self, key: str) -> Optional["ConfigFields"]:
        v, found = self._get(key, None, False)
        if not found:
            return None
        if not isinstance(v, dict):
            raise ConfigError(f"{self.origin}: key '{key}' is not an object")
        return ConfigFields(v, f"{self.origin}:{key}")
