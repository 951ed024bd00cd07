"""Kinds of parts by name.

A description (`tau_rs_b200.config.specs`) carries a `kind`; the class registered under
that kind builds the part from the description alone.  A new mixer, feed-forward, norm,
position encoding or block arrangement is added by registering a class here, from
anywhere: nothing else in the library names the kinds.
"""
from __future__ import annotations

from typing import Callable, Dict

_KINDS: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
}


def _register(family: str, kind: str):
    def decorate(cls):
        _KINDS[family][kind] = cls
        return cls
    return decorate


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_block(kind: str):
    return _register("block", kind)


def unregister(family: str, kind: str) -> None:
    _KINDS[family].pop(kind, None)


def build(family: str, spec, **context):
    """Builds the part that `spec.kind` names; `context` passes the prefix, dtype and device."""
    try:
        cls = _KINDS[family][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_KINDS[family])) or "none"
        raise KeyError(f"no {family} of kind {spec.kind!r} is registered (registered: {known})") from None
    return cls(spec, **context)
