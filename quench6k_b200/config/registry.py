"""One registry from an architecture's name (config.json `architectures[0]`) to its model.

The reference picks the Flint path by `general.architecture == "flint"`
(crates/engine/src/flint.rs:193-217, crates/cli/src/serve.rs:390-399).  Here an architecture is a
pair (config class, builder); the builder returns a spec.ModelSpec and nothing else of the
framework knows the architecture's name.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict


@dataclass
class Architecture:
    name: str
    config_cls: Any                       # has from_dict(dict) and to_dict()
    build_spec: Callable[[Any], Any]      # config -> spec.ModelSpec


_ARCHITECTURES: Dict[str, Architecture] = {}


class UnknownArchitecture(KeyError):
    pass


def register_architecture(name: str, config_cls: Any, build_spec: Callable[[Any], Any], aliases=()) -> None:
    arch = Architecture(name, config_cls, build_spec)
    for n in (name, *aliases):
        _ARCHITECTURES[n] = arch


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise UnknownArchitecture(
            f"unknown architecture {name!r}; registered: {', '.join(sorted(_ARCHITECTURES))}") from None


def known_architectures():
    return sorted(_ARCHITECTURES)


def read_config_dict(path: str) -> Dict[str, Any]:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        return json.load(f)


def architecture_of(config_dict: Dict[str, Any]) -> Architecture:
    names = config_dict.get("architectures")
    if not names or not isinstance(names, list):
        raise UnknownArchitecture("config.json has no 'architectures' list; registered: " + ", ".join(known_architectures()))
    return get_architecture(names[0])


def load_config(path: str):
    """(architecture, typed config) of a model folder or a config.json."""
    d = read_config_dict(path)
    arch = architecture_of(d)
    return arch, arch.config_cls.from_dict(d)
