"""Registries from a spec's `kind` to the class that builds it, one per sort of part.

A new mixer, feed-forward, norm, position encoding or block arrangement is added by registering a
class under a new kind and using that kind in a spec; nothing else in the package changes.
"""

from __future__ import annotations

from typing import Callable, Dict

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {},
    "feed_forward": {},
    "norm": {},
    "position": {},
    "block": {},
    "embedding": {},
    "head": {},
}


def register_part(sort: str, kind: str, factory: Callable, replace: bool = False) -> None:
    """`factory(spec, runtime)` builds the part.  sort: mixer, feed_forward, norm, position, block, embedding, head."""
    if sort not in _REGISTRIES:
        raise ValueError(f"unknown sort of part {sort!r}; known: {', '.join(_REGISTRIES)}")
    if kind in _REGISTRIES[sort] and not replace:
        raise ValueError(f"{sort} kind {kind!r} is already registered")
    _REGISTRIES[sort][kind] = factory


def unregister_part(sort: str, kind: str) -> None:
    _REGISTRIES[sort].pop(kind, None)


def build_part(sort: str, spec, runtime):
    kind = getattr(spec, "kind", None)
    table = _REGISTRIES[sort]
    if kind not in table:
        raise ValueError(f"no {sort} of kind {kind!r} is registered; known: {', '.join(sorted(table)) or 'none'}")
    return table[kind](spec, runtime)


def known_parts(sort: str):
    return sorted(_REGISTRIES[sort])
