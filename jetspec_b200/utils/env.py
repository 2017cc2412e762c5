"""Environment-variable flags.

The reference configures itself through constructor kwargs plus a handful of
``JETSPEC_*`` environment variables (``jetspec/inference_engine/engine.py:80-89``,
``:295``, ``:1098``, ``:49``).  The same variable names are honoured here.
"""
from __future__ import annotations

import os

_TRUE = {"1", "true", "yes", "on"}
_FALSE = {"0", "false", "no", "off", ""}


def env_flag(name: str, default: bool = False) -> bool:
    """True when ``name`` is set to a truthy string; ``default`` when unset."""
    raw = os.environ.get(name)
    if raw is None:
        return default
    return raw.strip().lower() in _TRUE


def env_flag_enabled(name: str, default: bool = True) -> bool:
    """Default-on flag: only an explicit falsy value turns it off."""
    raw = os.environ.get(name)
    if raw is None:
        return default
    return raw.strip().lower() not in _FALSE


def env_int(name: str, default: int) -> int:
    raw = os.environ.get(name)
    if raw is None or not raw.strip():
        return default
    return int(raw)


def env_str(name: str, default: str = "") -> str:
    return os.environ.get(name, default)
