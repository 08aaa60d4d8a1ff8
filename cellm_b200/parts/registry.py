"""Registries of part kinds. A new mixer, feed-forward, norm, position
encoding, block arrangement, embedding or head is one class and one `register_*` call; nothing
else in the package names the kinds."""
from __future__ import annotations

from ..config.errors import ConfigError

_REGISTRIES: dict[str, dict[str, type]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
                                           "embedding": {}, "head": {}}


def _register(family: str, kind: str, cls: type) -> type:
    cls.kind = kind
    _REGISTRIES[family][kind] = cls
    return cls


def register_mixer(kind, cls): return _register("mixer", kind, cls)
def register_feed_forward(kind, cls): return _register("feed_forward", kind, cls)
def register_norm(kind, cls): return _register("norm", kind, cls)
def register_position(kind, cls): return _register("position", kind, cls)
def register_block(kind, cls): return _register("block", kind, cls)
def register_embedding(kind, cls): return _register("embedding", kind, cls)
def register_head(kind, cls): return _register("head", kind, cls)


def part_class(family: str, kind: str) -> type:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        raise ConfigError(f"no {family} part of kind {kind!r} is registered; "
                          f"known: {sorted(_REGISTRIES[family])}") from None


def registered(family: str) -> list[str]:
    return sorted(_REGISTRIES[family])
