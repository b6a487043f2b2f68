"""One registry from an architecture's name to what builds its model.

The reference walks a table of ``BnModelArchOps`` and takes the first entry whose
predicate matches the GGUF architecture string (src/model_arch.c:862-987).  Here
the key is ``config.json``'s ``architectures[0]`` and an unknown name is an error
that lists the known ones.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict

from .spec import ConfigError, ModelSpec


@dataclass(frozen=True)
class Architecture:
    """What an architecture supplies.

    ``read_config(dict)`` returns the typed configuration; ``to_spec(config)``
    translates it into the block-by-block ``ModelSpec``; ``tensor_name(path)``
    gives the checkpoint tensor name of a parameter path such as
    ``blocks.0.mixer.q``; ``cap_positions(config, n)`` applies ``--maxseq``.
    """

    name: str
    read_config: Callable[[Dict[str, Any]], Any]
    to_spec: Callable[[Any], ModelSpec]
    tensor_name: Callable[[str], str]
    cap_positions: Callable[[Any, int], Any]
    config_to_dict: Callable[[Any], Dict[str, Any]]


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    if arch.name in _ARCHITECTURES:
        raise ConfigError(f"architecture '{arch.name}' is registered twice")
    _ARCHITECTURES[arch.name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def known_architectures():
    return sorted(_ARCHITECTURES)


def architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture '{name}'; known: {', '.join(known_architectures())}") from None


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json") if os.path.isdir(model_dir) else model_dir
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at '{path}'")
    with open(path, "r", encoding="utf-8") as f:
        try:
            d = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"'{path}' is not valid JSON: {e}") from None
    if not isinstance(d, dict):
        raise ConfigError(f"'{path}' must hold a JSON object")
    return d


def architecture_of(config_dict: Dict[str, Any]) -> Architecture:
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)) or not isinstance(archs[0], str):
        raise ConfigError("config.json has no 'architectures' list; known: "
                          + ", ".join(known_architectures()))
    return architecture(archs[0])
