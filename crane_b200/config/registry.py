"""One registry from an architecture's name to its configuration class and to
the function that lays the model out as a ``ModelSpec``.

Lookup follows the reference's detection order
(crane-serve/src/engine/model_factory.rs:100-180): an explicit model type,
then ``architectures`` of config.json, then ``model_type``; names are matched
without regard to case.  Unlike the reference (model_factory.rs:174-178: falls
back to another model with a warning) an unknown architecture is an error that
lists what is registered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

from .spec import ModelSpec


class UnknownArchitecture(KeyError):
    def __str__(self) -> str:          # KeyError would quote the message
        return self.args[0] if self.args else ""


@dataclass
class Architecture:
    name: str
    aliases: List[str]
    config_from_dict: Callable[[Dict[str, Any]], Any]
    build_spec: Callable[[Any], ModelSpec]


_ARCHS: Dict[str, Architecture] = {}
_ALIASES: Dict[str, str] = {}


def register_architecture(name: str, config_from_dict, build_spec, aliases=()) -> Architecture:
    """Register (or replace) an architecture under its config.json name."""
    arch = Architecture(name, [a.lower() for a in aliases], config_from_dict, build_spec)
    _ARCHS[name.lower()] = arch
    for a in arch.aliases:
        _ALIASES[a] = name.lower()
    return arch


def registered() -> List[str]:
    return sorted(a.name for a in _ARCHS.values())


def _lookup(key: Optional[str]) -> Optional[Architecture]:
    if not key:
        return None
    k = key.lower()
    if k in _ARCHS:
        return _ARCHS[k]
    if k in _ALIASES:
        return _ARCHS[_ALIASES[k]]
    return None


def resolve(config: Dict[str, Any], model_type: Optional[str] = None) -> Architecture:
    """The architecture of a config.json dict; ``model_type`` is a user's hint
    ("auto" or empty: none), as the reference's ``--model-type``."""
    hint = None if not model_type or model_type.lower() == "auto" else model_type
    tried: List[str] = []
    if hint:
        tried.append(hint)
        arch = _lookup(hint)
        if arch is None:
            raise UnknownArchitecture(
                f"model type '{hint}' is not registered; registered: {', '.join(registered())}")
        return arch
    for a in config.get("architectures") or []:
        tried.append(str(a))
        arch = _lookup(str(a))
        if arch is not None:
            return arch
    mt = config.get("model_type")
    if mt:
        tried.append(str(mt))
        arch = _lookup(str(mt))
        if arch is not None:
            return arch
    raise UnknownArchitecture(
        "no registered architecture for config.json (tried: " + (", ".join(tried) or "nothing")
        + "); registered: " + ", ".join(registered()))
