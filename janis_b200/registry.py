"""One registry from an architecture's name to its configuration class and model builder.

The reference picks the model with a switch on config.json's `model_type`
(`engine.go:153-205`) and answers `unsupported model_type %q` for anything else
(`engine.go:204`).  Here the key is `architectures[0]` (for example
"Gemma2ForCausalLM"), with `model_type` as the fallback, and new architectures
are added by calling `register_architecture`, from inside the package or from
a user's own code.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .config.base import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any                   # has from_dict(raw, where) and to_dict()
    build: Callable[..., Any]           # build(config) -> engine.model.DecoderModel
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build: Callable[..., Any],
                          model_types: tuple[str, ...] = (), replace: bool = False) -> Architecture:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    arch = Architecture(name, config_class, build, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve(raw: Mapping[str, Any], where: str = "config.json") -> Architecture:
    """The architecture that a parsed config.json names."""
    names = raw.get("architectures") or []
    if isinstance(names, str):
        names = [names]
    for n in names:
        if n in _ARCHITECTURES:
            return _ARCHITECTURES[n]
    mt = raw.get("model_type")
    for arch in _ARCHITECTURES.values():
        if mt is not None and mt in arch.model_types:
            return arch
    if names:
        raise ConfigError(f"{where}: unsupported architecture {names[0]!r} "
                          f"(registered: {', '.join(architectures()) or 'none'})")
    raise ConfigError(f"{where}: unsupported model_type {mt!r} "
                      f"(registered: {', '.join(architectures()) or 'none'})")
