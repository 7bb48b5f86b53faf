"""Helpers for configurations that are nested objects (a list of layers, each with its mixer's and its
feed-forward's sizes): typed reads whose errors name the key by its path."""
from __future__ import annotations

from typing import Any, Dict

from ..errors import ErrorCode, PhotonError


def bad(msg: str) -> PhotonError:
    return PhotonError(ErrorCode.INVALID_CONFIG, "config.json: " + msg)


def num(d: Dict[str, Any], key: str, where: str, kind=int, positive: bool = True, default=None):
    if not isinstance(d, dict):
        raise bad(f"'{where}' must be an object")
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise bad(f"required key '{where}.{key}' is missing")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and not isinstance(v, int)):
        raise bad(f"key '{where}.{key}' must be {'an integer' if kind is int else 'a number'}, got {v!r}")
    v = kind(v)
    if positive and not v > 0:
        raise bad(f"key '{where}.{key}' must be positive, got {v!r}")
    return v


def obj(d: Any, key: str, where: str, required: bool = False) -> Any:
    """The object under ``key`` (None when absent or null and not required)."""
    if not isinstance(d, dict):
        raise bad(f"'{where}' must be an object")
    v = d.get(key)
    if v is None:
        if required:
            raise bad(f"required key '{where}.{key}' is missing")
        return None
    if not isinstance(v, dict):
        raise bad(f"'{where}.{key}' must be an object")
    return v
