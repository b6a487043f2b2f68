"""Registries from a spec's ``kind`` to the class that builds the part.

``@register_mixer("attention")`` and its siblings add a class; ``build_part`` looks a
spec up by the role it plays and its ``kind``.  A new mixer, feed-forward, norm,
position encoding, block arrangement or output head is one class with one decorator;
nothing else in the library has to change.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Type

from ..config.spec import ConfigError
from .base import BuildContext, Part

_REGISTRIES: Dict[str, Dict[str, Type[Part]]] = {
    "mixer": {}, "ffn": {}, "norm": {}, "position": {}, "block": {}, "head": {},
}


def _register(role: str, kind: str) -> Callable[[Type[Part]], Type[Part]]:
    def deco(cls: Type[Part]) -> Type[Part]:
        table = _REGISTRIES[role]
        if kind in table and table[kind] is not cls:
            raise ConfigError(f"{role} kind '{kind}' is registered twice")
        table[kind] = cls
        return cls
    return deco


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_ffn(kind: str):
    return _register("ffn", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_block(kind: str):
    return _register("block", kind)


def register_head(kind: str):
    return _register("head", kind)


def unregister(role: str, kind: str) -> None:
    _REGISTRIES[role].pop(kind, None)


def known(role: str):
    return sorted(_REGISTRIES[role])


def build_part(role: str, spec: Any, build: BuildContext) -> Part:
    kind = getattr(spec, "kind", None)
    table = _REGISTRIES[role]
    if kind not in table:
        raise ConfigError(f"no {role} of kind {kind!r}; known: {', '.join(sorted(table)) or '(none)'}")
    return table[kind](spec, build)
