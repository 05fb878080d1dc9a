"""Registries of part kinds: mixers, feed-forwards, norms, position encodings, blocks.

A part class is registered under the ``kind`` that a :class:`PartSpec` names.  Code outside the
package (a test, a plug-in) registers its own kinds the same way; nothing in the framework
lists the kinds it knows.
"""
from __future__ import annotations

from typing import Callable

from .spec import PartSpec


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict[str, type] = {}

    def register(self, kind: str, cls: type | None = None, *, replace: bool = False):
        def deco(c):
            if kind in self._kinds and not replace and self._kinds[kind] is not c:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = c
            return c

        return deco(cls) if cls is not None else deco

    def unregister(self, kind: str):
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._kinds[kind]
        except KeyError:
            known = ", ".join(sorted(self._kinds)) or "none"
            raise KeyError(f"unknown {self.what} kind {kind!r}; registered: {known}") from None

    def build(self, spec: PartSpec, **extra):
        return self.get(spec.kind)(spec, **extra)

    def kinds(self):
        return sorted(self._kinds)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")

register_mixer: Callable = MIXERS.register
register_feed_forward: Callable = FEED_FORWARDS.register
register_norm: Callable = NORMS.register
register_position: Callable = POSITIONS.register
register_block: Callable = BLOCKS.register
