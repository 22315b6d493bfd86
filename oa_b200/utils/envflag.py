"""Environment knobs (Source/Public/Oa/Core/EnvFlag.h:10-67): IsSet / GetString / GetInt / SetIfUnset."""
from __future__ import annotations

import os

_FALSE = {"", "0", "false", "off", "no"}


def IsSet(name: str) -> bool:
    v = os.environ.get(name)
    return v is not None and v.strip().lower() not in _FALSE


def GetString(name: str, default: str = "") -> str:
    return os.environ.get(name, default)


def GetInt(name: str, default: int = 0) -> int:
    try:
        return int(os.environ.get(name, default))
    except (TypeError, ValueError):
        return default


def GetFloat(name: str, default: float = 0.0) -> float:
    try:
        return float(os.environ.get(name, default))
    except (TypeError, ValueError):
        return default


def SetIfUnset(name: str, value: str) -> None:
    os.environ.setdefault(name, value)


def ApplyNumericMode(mode: int) -> None:
    """Numeric mode -> knobs (Source/Public/Oa/Core/EnvFlag.h:73-83): Deterministic pins fixed-order reductions."""
    if int(mode) >= 1:
        SetIfUnset("OA_STABLE_MATH", "1")
    if int(mode) >= 2:
        SetIfUnset("OA_DETERMINISTIC", "1")
