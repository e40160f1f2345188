"""What every part of a layer is, and what a step hands to it.

A model is put together from parts: an embedding, blocks (each an arrangement
of a mixer, a feed-forward and norms), a final norm and an output head.  A part
gets its sizes and constants as constructor arguments and the checkpoint names
of its tensors as a mapping; it never asks which model it is in.

Interfaces (all tensors are on the device; T = tokens of this step, packed
sequence after sequence without padding):

* `Part.tensor_specs()` -> {checkpoint name: TensorSpec}: what it loads.
* `Part.load(store, rt)`: take its tensors from the store (`store.get(name,
  dtype)`), fuse or widen them as its kernels want.
* `Norm.forward(x, ctx, out, rows=None)`; `Norm.residual_add(h, r, ctx,
  next_norm=None, out=None)`: h += norm(r) on the float32 residual stream, and
  out = next_norm(h) when asked.
* `PositionEncoding.encode(qkv, ctx, nq, nkv, hd, with_keys)`: encode queries
  (and keys) in place; `encode_and_store(qkv, ctx, nq, nkv, hd, kv_line)`: the
  same and write keys and values into the cache line (by default `encode`
  followed by the plain store; an encoding with a fused kernel overrides it).
* `Mixer.cache_needs()` -> {name: KVNeed | StateNeed}; `Mixer.forward(x, ctx,
  line)` -> [T, hidden] in the activation dtype.  `line[name]` is the cache part
  it asked for; `line.write` is False when the schedule lets it only read.
* `FeedForward.forward(x, ctx)` -> [T, hidden].
* `Block.forward(h, ctx, line, y_in=None, next_norm=None)` -> (h, y_next): h is the
  float32 residual stream, updated in place; y_in is this block's first norm
  already applied (by the block before), y_next is `next_norm` applied to the
  result, so that a norm can be fused across the border of two blocks.

The reference writes each model against its tensor-op interface
(`engine/backend.go:142-287`) with a struct per layer kind holding its constants
(`gemma/gemma.go:31-35`, `:98-100`, `:127-131`); the split into exchangeable
parts chosen layer by layer is this library's.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch

from ..weights.loader import TensorSpec


class Runtime:
    """The compute dtype, the device and the kernels a model runs with."""

    def __init__(self, dtype: torch.dtype, device, ops):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, found {dtype}")
        self.dtype = dtype
        self.device = device
        self.ops = ops
        dev = torch.device(device)
        self.sm_count = (torch.cuda.get_device_properties(dev).multi_processor_count
                         if dev.type == "cuda" else 1)

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """out = x w^T in the compute dtype, accumulated in float32."""
        if self.dtype == torch.float32:
            return self.ops.gemm_f32(x, w, out)
        return self.ops.linear_bf16(x, w, out)


class Workspace:
    """Named device buffers that live across steps (nothing is allocated in a
    steady state, which stream capture needs).  `buf` returns a view of the
    first rows; a buffer grows when a larger one is asked for."""

    def __init__(self, device):
        self.device = device
        self._bufs: dict[str, torch.Tensor] = {}
        self.frozen = False
        self._in_graph: set[str] = set()          # names whose current buffer a CUDA graph has recorded
        self._retired: list[torch.Tensor] = []    # outgrown buffers that a graph still writes to
        self._views: dict[str, tuple] = {}        # name -> (shape, buffer, view): the view handed out last

    def buf(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        shape = tuple(shape)
        last = self._views.get(name)
        if last is not None and last[0] == shape and last[1].dtype == dtype and last[1] is self._bufs.get(name):
            if self.frozen:
                self._in_graph.add(name)
            return last[2]                        # the same view as last step: no tensor objects to build
        n = 1
        for s in shape:
            n *= int(s)
        cur = self._bufs.get(name)
        if cur is None or cur.dtype != dtype or cur.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow during stream capture")
            if cur is not None and name in self._in_graph:
                self._retired.append(cur)         # keep its memory valid for the graphs that recorded it
                self._in_graph.discard(name)
            # zeros, not whatever the allocator hands out: a kernel that reads a row nobody wrote (a tile that runs
            # past the step's rows) must find numbers there
            cur = torch.zeros(max(n, 1), dtype=dtype, device=self.device)
            self._bufs[name] = cur
        if self.frozen:
            self._in_graph.add(name)
        view = cur[:n].view(*shape)
        self._views[name] = (shape, cur, view)
        return view

    def fill(self, value) -> None:
        """Every buffer filled with `value` (tests poison the workspace with NaN between steps: a step must write
        what it reads)."""
        for t in self._bufs.values():
            if t.is_floating_point():
                t.fill_(value)

    def begin_capture(self) -> None:
        self.frozen = True

    def end_capture(self) -> None:
        self.frozen = False

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


@dataclass
class StepContext:
    """One step's batch as the parts see it."""
    rt: Runtime
    ws: Workspace
    mode: str                       # "prefill": one or more tokens a sequence, packed; "decode": one token each
    n_tok: int
    n_seq: int
    tokens: torch.Tensor            # int32 [T]
    tok_pos: torch.Tensor           # int32 [T] absolute position of each token
    tok_seq: torch.Tensor           # int32 [T] index of its sequence in this step
    seq_slot: torch.Tensor          # int32 [n_seq] cache slot, < 0 for padding
    seq_start: torch.Tensor         # int32 [n_seq] tokens cached before the step
    seq_end: torch.Tensor           # int32 [n_seq] tokens cached after the step
    seq_first_row: torch.Tensor     # int32 [n_seq] row of the sequence's first token of this step in the packed step
    len_bound: int = 0              # host-side bound on max(seq_end); sizes the decode grids
    len_mean: int = 0               # host-side estimate of mean(seq_end) over the step's rows, rounded up to an eighth of
                                    # len_bound (0: unknown, take len_bound); it tunes launch shapes and changes no result
    len_even: bool = True           # whether the sequences are about equally long (the shortest at least 3/4 of the longest)
    step_lens: tuple | None = None  # host-side: the tokens each sequence brings to a "prefill" step, when the step's tables
                                    # hold just these (None in a step recorded for other lengths too); launch shapes only
    extends: bool = False           # a "prefill" step some of whose sequences have tokens in the cache already
                                    # (seq_start > 0): a mixer reads those from its cache line and stores this
                                    # step's own only after it has attended
    shared: dict = field(default_factory=dict)   # scratch that parts of one step hand to each other


class Part:
    # False for a part whose step cannot be recorded into a CUDA graph (it synchronises, allocates by
    # data-dependent sizes, or copies from the host); steps are then launched kernel by kernel.  A part that
    # leaves it True meets padding in recorded steps, decode and prompt steps alike: sequences whose slot is
    # negative (and the tokens that name them) must be stored nowhere and must change no other row.
    graph_safe = True

    def tensor_specs(self) -> dict[str, TensorSpec]:
        return {}

    def load(self, store, rt: Runtime) -> None:
        pass

    def sub_parts(self) -> list["Part"]:
        return []


class Norm(Part):
    def forward(self, x, ctx: StepContext, out, rows=None):
        raise NotImplementedError

    def residual_add(self, h, r, ctx: StepContext, next_norm: "Norm | None" = None, out=None):
        raise NotImplementedError


class PositionEncoding(Part):
    def encode(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, with_keys: bool):
        """Encode the queries of qkv [T, heads, hd] (and the keys behind them when with_keys) in place; store
        nothing.  A step that continues sequences attends before it stores, so it needs the two apart."""
        raise NotImplementedError(f"{type(self).__name__} has no encode(): it cannot take a step that continues "
                                  "sequences with several tokens")

    def encode_and_store(self, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        own = kv_line is not None and kv_line.write
        self.encode(qkv, ctx, nq, nkv, hd, own)
        if own:
            ctx.rt.ops.kv_store(qkv, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, ctx.seq_end, nq, nkv, hd, kv_line.k,
                                kv_line.v, kv_line.table, kv_line.ring_len)
        return qkv

    def project_encode_store(self, x, w, qkv, ctx: StepContext, nq: int, nkv: int, hd: int, kv_line):
        """qkv [T, heads, hd] = x w^T, then encode_and_store.  An encoding whose kernels can do all of it at once
        overrides this; the result must be what this order of the two leaves in the queries and in the cache."""
        ctx.rt.linear(x, w, qkv.view(qkv.shape[0], -1))
        return self.encode_and_store(qkv, ctx, nq, nkv, hd, kv_line)


class Mixer(Part):
    def cache_needs(self) -> Mapping[str, Any]:
        return {}

    def prompt_flops(self, n_tokens: int) -> float:
        """Floating-point operations of a prompt of n_tokens from position 0 beyond the products with the part's
        weight matrices (for attention: scores and weighted sums over the keys each query sees).  Measurement
        asks the mixer, so that it counts another mixer's work as well as attention's."""
        return 0.0

    def forward(self, x, ctx: StepContext, line):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, ctx: StepContext):
        raise NotImplementedError


class Block(Part):
    first_norm: Norm | None = None
    mixer: Mixer

    def forward(self, h, ctx: StepContext, line, y_in=None, next_norm: Norm | None = None):
        raise NotImplementedError


class WeightStore:
    """Loaded tensors by checkpoint name, with conversions cached so that parts
    that share a tensor (a tied head) share its converted copy too."""

    def __init__(self, tensors: Mapping[str, torch.Tensor]):
        self._raw = dict(tensors)
        self._conv: dict[tuple[str, torch.dtype], torch.Tensor] = {}

    def get(self, name: str, dtype: torch.dtype | None = None) -> torch.Tensor:
        try:
            t = self._raw[name]
        except KeyError:
            raise KeyError(f"tensor {name!r} is not in the store (never loaded, or given up by the part that "
                           "fused it into a layout of its own)") from None
        if dtype is None or t.dtype == dtype:
            return t
        key = (name, dtype)
        if key not in self._conv:
            self._conv[key] = t.to(dtype)
        return self._conv[key]

    def drop(self, *names: str) -> None:
        """Forget the stored form (and its conversions) of tensors whose only user keeps a fused copy: a model
        must not sit in memory twice once it is loaded."""
        for name in names:
            self._raw.pop(name, None)
            for key in [k for k in self._conv if k[0] == name]:
                del self._conv[key]

    def names(self):
        return list(self._raw)
