"""Named plugins: a family of plugins is a subclass of :class:`Plugin`; each family keeps its own table of
``name -> {method -> function}``, functions join it through a decorator, and an instance made with a name calls
them.  The data engine's record converters are one family (``DataConverter``); users add their own formats with
``@DataConverter("my_format").register()`` and name them in the dataset description.

Reference: ``v1/utils/plugin.py:26-92`` (one shared table keyed by name; here each family has its own table, so two
families may use the same plugin name)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List

MAIN = "__call__"


class Plugin:
    _tables: Dict[type, Dict[str, Dict[str, Callable]]] = {}

    def __init__(self, name: str | None = None) -> None:
        self.name = name

    @classmethod
    def _table(cls) -> Dict[str, Dict[str, Callable]]:
        return Plugin._tables.setdefault(cls, {})

    @classmethod
    def names(cls) -> List[str]:
        return sorted(cls._table())

    @classmethod
    def has(cls, name: str, method: str = MAIN) -> bool:
        return method in cls._table().get(name, {})

    def register(self, method: str = MAIN, *, replace: bool = False) -> Callable[[Callable], Callable]:
        if not self.name:
            raise ValueError("a plugin needs a name before functions can be registered under it")
        slots = self._table().setdefault(self.name, {})
        if method in slots and not replace:
            raise ValueError(f"{type(self).__name__} '{self.name}' already has '{method}'; pass replace=True to override")

        def deco(fn: Callable) -> Callable:
            slots[method] = fn
            return fn

        return deco

    def __getitem__(self, method: str) -> Callable:
        try:
            return self._table()[self.name][method]
        except KeyError:
            raise KeyError(f"{type(self).__name__} '{self.name}' has no '{method}' "
                           f"(known plugins: {', '.join(self.names()) or 'none'})") from None

    def __getattr__(self, method: str) -> Callable:
        if method.startswith("_"):
            raise AttributeError(method)
        try:
            return self[method]
        except KeyError as e:
            raise AttributeError(str(e)) from None

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        return self[MAIN](*args, **kwargs)


class DataConverter(Plugin):
    """``DataConverter(name)(record) -> {"messages": [...], ...}``."""


class BatchingStrategy(Plugin):
    """``BatchingStrategy(name)(rows, generator) -> list of micro-batches``; the built-in strategies are methods of
    ``BatchGenerator`` and user strategies are looked up here."""
