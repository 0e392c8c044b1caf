"""Name -> object registries: the one place a config string becomes a callable.

Mirrors the behaviour of the reference registry (`src/kohakumoss_common/registry.py:13,47`):
a value may be a registered name, a dotted import path, or a dict
`{"name": ..., **kwargs}`.
"""

from __future__ import annotations

import difflib
import importlib
from collections.abc import Callable
from typing import Any


class Registry:
    def __init__(self, kind: str):
        self.kind = kind
        self._items: dict[str, Any] = {}

    def register(self, name: str, obj: Any = None):
        if obj is not None:
            self._items[name] = obj
            return obj

        def deco(fn):
            self._items[name] = fn
            return fn

        return deco

    def names(self) -> tuple[str, ...]:
        return tuple(sorted(self._items))

    def __contains__(self, name: str) -> bool:
        return name in self._items

    def get(self, name: str) -> Any:
        if name in self._items:
            return self._items[name]
        if "." in name:
            module, _, attr = name.rpartition(".")
            return getattr(importlib.import_module(module), attr)
        hint = difflib.get_close_matches(name, self._items, n=3)
        tail = f"; did you mean {', '.join(hint)}?" if hint else ""
        raise KeyError(f"unknown {self.kind} {name!r} (have: {', '.join(self.names())}){tail}")


def build(registry: Registry, spec: str | dict | Callable, **defaults) -> Any:
    """Instantiate `spec` (name, dotted path, dict with `name`, or a ready object)."""
    if isinstance(spec, str):
        return registry.get(spec)(**defaults)
    if isinstance(spec, dict):
        kwargs = {**defaults, **{k: v for k, v in spec.items() if k != "name"}}
        return registry.get(spec["name"])(**kwargs)
    return spec
