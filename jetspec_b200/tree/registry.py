"""Name → algorithm registry (``register_tree_algo`` / ``get_algorithm`` / ``list_algorithms``), the public
contract of ``jetspec/tree/_core/registry.py:18-39``."""
from __future__ import annotations

from .types import TreeAlgorithm

_ALGOS: dict = {}


def register_tree_algo(name: str):
    def wrap(cls):
        if name in _ALGOS:
            raise ValueError(f"tree algorithm {name!r} already registered")
        cls.name = name
        _ALGOS[name] = cls
        return cls
    return wrap


def get_algorithm(name: str, **init_kwargs) -> TreeAlgorithm:
    try:
        cls = _ALGOS[name]
    except KeyError:
        raise KeyError(f"unknown tree algorithm {name!r}. Available: {sorted(_ALGOS)}") from None
    return cls(**init_kwargs)


def list_algorithms() -> list:
    return sorted(_ALGOS)
