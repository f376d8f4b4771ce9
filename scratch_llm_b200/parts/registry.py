"""Registries of parts, keyed by the ``kind`` of a :class:`~scratch_llm_b200.config.spec.PartSpec`.

Adding a part: write a class with the interface of :mod:`scratch_llm_b200.parts.base`, and
register it under a new key; a configuration then names the key layer by layer.  Nothing else
in the framework changes.
"""

from __future__ import annotations

from typing import Any, Callable

MIXERS: dict[str, Callable[..., Any]] = {}
FEED_FORWARDS: dict[str, Callable[..., Any]] = {}
NORMS: dict[str, Callable[..., Any]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., Any]] = {}
BLOCKS: dict[str, Callable[..., Any]] = {}


def _register(table: dict[str, Callable[..., Any]], what: str):
    def register(kind: str, factory: Callable[..., Any] | None = None):
        def put(f):
            if kind in table:
                raise ValueError(f"{what} {kind!r} is already registered")
            table[kind] = f
            return f
        return put(factory) if factory is not None else put
    return register


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")


def make(table: dict[str, Callable[..., Any]], what: str, spec) -> Any:
    try:
        factory = table[spec.kind]
    except KeyError:
        known = ", ".join(sorted(table)) or "(none)"
        raise ValueError(f"unknown {what} {spec.kind!r}; registered: {known}") from None
    return factory(**dict(spec.args))
