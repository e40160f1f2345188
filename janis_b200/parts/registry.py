"""Kinds of parts by name, so that a configuration can choose them layer by layer.

An architecture's builder looks a kind up with `make(family, kind, **params)`;
a user's code can add kinds of its own with `register(family, kind, factory)`
and use them from a builder of its own, without touching this package.
"""
from __future__ import annotations

from typing import Any, Callable

FAMILIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")

_KINDS: dict[str, dict[str, Callable[..., Any]]] = {f: {} for f in FAMILIES}


def register(family: str, kind: str, factory: Callable[..., Any], replace: bool = False) -> None:
    if family not in _KINDS:
        raise ValueError(f"unknown family of parts {family!r} (families: {', '.join(FAMILIES)})")
    if kind in _KINDS[family] and not replace:
        raise ValueError(f"{family} kind {kind!r} is already registered")
    _KINDS[family][kind] = factory


def unregister(family: str, kind: str) -> None:
    _KINDS.get(family, {}).pop(kind, None)


def kinds(family: str) -> tuple[str, ...]:
    return tuple(sorted(_KINDS[family]))


def make(family: str, kind: str, **params):
    try:
        factory = _KINDS[family][kind]
    except KeyError:
        raise ValueError(f"unknown {family} kind {kind!r} (registered: {', '.join(kinds(family)) or 'none'})") from None
    return factory(**params)


def _register_builtin() -> None:
    from .attention import SoftmaxAttention
    from .block import PreNormBlock, SandwichBlock
    from .embedding import Embedding, LMHead
    from .feedforward import GatedMLP
    from .norm import RMSNorm
    from .position import NoPosition, RotaryEncoding

    register("mixer", "softmax_attention", SoftmaxAttention)
    register("feed_forward", "gated_mlp", GatedMLP)
    register("norm", "rms_norm", RMSNorm)
    register("position", "rotary", RotaryEncoding)
    register("position", "none", NoPosition)
    register("block", "sandwich", SandwichBlock)
    register("block", "pre_norm", PreNormBlock)
    register("embedding", "scaled_table", Embedding)       # rows of a table times a constant (1 for most models)
    register("head", "capped_linear", LMHead)              # y W^T, tied to the embedding's table or not, then an optional cap


_register_builtin()
