"""A decoder put together from parts, and the order its layers run in.

`DecoderModel` holds an embedding, a list of blocks, a *schedule*, a final norm
and an output head.  The schedule is data: a list of `LayerCall(layer,
cache_line, write)`.  It may name a layer twice (a looped layer, each visit with
a cache line of its own or a shared one) and may let a layer read the cache line
that another entry writes (`write=False`: the layer projects queries only).
Every cache line is written by exactly one entry, which comes before its readers.

The reference runs its blocks in list order with one cache per block
(`gemma/gemma.go:204-206`); its looped decoder visits layers repeatedly
(`inkling2/`), and its hybrid model picks the cache kind per layer
(`qwen35/model.go:153-169`).  The last position alone is projected to logits
there (`gemma/gemma.go:207-212`); here the rows to project are given.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from ..parts.base import Block, Norm, Part, Runtime, StepContext
from ..weights.loader import TensorSpec


@dataclass(frozen=True)
class LayerCall:
    layer: int
    cache_line: int
    write: bool = True


def _walk(part: Part):
    yield part
    for sub in part.sub_parts():
        yield from _walk(sub)


class DecoderModel:
    def __init__(self, config, embedding: Part, blocks: Sequence[Block], final_norm: Norm, head: Part,
                 schedule: Sequence[LayerCall] | None = None, ignorable_tensors: Sequence[str] = (),
                 stop_tokens: Sequence[int] = (), max_context: int = 8192):
        self.config = config
        self.embedding = embedding
        self.blocks = list(blocks)
        self.final_norm = final_norm
        self.head = head
        self.schedule = list(schedule) if schedule is not None else [LayerCall(i, i) for i in range(len(blocks))]
        self.ignorable_tensors = tuple(ignorable_tensors)
        self.stop_tokens = tuple(stop_tokens)
        self.max_context = int(max_context)
        self.hidden = embedding.hidden
        self.vocab = head.vocab
        self._check_schedule()
        self.graph_safe = all(getattr(p, "graph_safe", True) for p in self.parts())

    def _check_schedule(self) -> None:
        if not self.schedule:
            raise ValueError("the layer schedule is empty")
        n_lines = 1 + max(c.cache_line for c in self.schedule)
        writer: dict[int, int] = {}
        self.readers: dict[int, int] = {i: 0 for i in range(n_lines)}
        for idx, c in enumerate(self.schedule):
            if not 0 <= c.layer < len(self.blocks):
                raise ValueError(f"schedule entry {idx} names layer {c.layer}; there are {len(self.blocks)}")
            if c.cache_line < 0:
                raise ValueError(f"schedule entry {idx} names a negative cache line")
            if c.write:
                if c.cache_line in writer:
                    raise ValueError(f"cache line {c.cache_line} is written by schedule entries "
                                     f"{writer[c.cache_line]} and {idx}")
                writer[c.cache_line] = idx
            else:
                if c.cache_line not in writer:
                    raise ValueError(f"schedule entry {idx} reads cache line {c.cache_line} before it is written")
                w = self.blocks[self.schedule[writer[c.cache_line]].layer].mixer.cache_needs()
                if dict(self.blocks[c.layer].mixer.cache_needs()) != dict(w):
                    raise ValueError(f"schedule entry {idx} reads cache line {c.cache_line}, whose writer "
                                     "keeps something else")
                self.readers[c.cache_line] += 1
        for line in range(n_lines):
            if line not in writer:
                raise ValueError(f"cache line {line} is never written")
        self.n_cache_lines = n_lines
        self._writer = writer

    # -- tensors -------------------------------------------------------------
    def parts(self):
        seen = set()
        for top in [self.embedding, *self.blocks, self.final_norm, self.head]:
            for p in _walk(top):
                if id(p) not in seen:
                    seen.add(id(p))
                    yield p

    def tensor_specs(self) -> dict[str, TensorSpec]:
        specs: dict[str, TensorSpec] = {}
        for p in self.parts():
            for name, spec in p.tensor_specs().items():
                if name in specs and specs[name].shape != spec.shape:
                    raise ValueError(f"tensor {name!r} is wanted with shapes {specs[name].shape} and {spec.shape}")
                specs.setdefault(name, spec)
        return specs

    def load(self, store, rt: Runtime) -> None:
        for top in [self.embedding, *self.blocks, self.final_norm, self.head]:
            self._load(top, store, rt, set())

    def _load(self, part: Part, store, rt, done: set) -> None:
        if id(part) in done:
            return
        done.add(id(part))
        part.load(store, rt)
        for sub in part.sub_parts():
            self._load(sub, store, rt, done)

    def cache_line_needs(self) -> list[dict]:
        return [dict(self.blocks[self.schedule[self._writer[line]].layer].mixer.cache_needs())
                for line in range(self.n_cache_lines)]

    # -- a step ----------------------------------------------------------------
    def forward(self, ctx: StepContext, cache) -> torch.Tensor:
        """Run the schedule over the step's tokens; returns the residual stream [T, hidden] float32."""
        h = ctx.ws.buf("stream.h", (ctx.n_tok, self.hidden), torch.float32)
        self.embedding.forward(ctx.tokens, ctx, h)
        y = None
        for idx, call in enumerate(self.schedule):
            blk = self.blocks[call.layer]
            nxt = self.blocks[self.schedule[idx + 1].layer].first_norm if idx + 1 < len(self.schedule) else None
            line = cache.line(call.cache_line, call.write, has_readers=call.write and self.readers[call.cache_line] > 0)
            h, y = blk.forward(h, ctx, line, y_in=y, next_norm=nxt)
        for late in ctx.shared.pop("after_step", ()):    # what parts put off until every layer has run
            late()
        return h

    def logits(self, ctx: StepContext, h: torch.Tensor, rows: torch.Tensor | None, n_rows: int,
               out: torch.Tensor) -> torch.Tensor:
        """Final norm and head over the given rows of h (all rows when `rows` is None) -> float32 [R, vocab]."""
        y = ctx.ws.buf("head.y", (n_rows, self.hidden), ctx.rt.dtype)
        self.final_norm.forward(h, ctx, y, rows)
        return self.head.forward(y, ctx, out)
