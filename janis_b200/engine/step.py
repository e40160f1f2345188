"""The step function: a batch of sequences, the tokens it is given, logits back.

A step is either a *prompt step* (every sequence of the batch is new and brings
its whole prompt; lengths may differ) or a *decode step* (every sequence brings
exactly one token).  The step runs only the tokens it is given, packed without
padding, against what earlier steps left in the cache, and returns float32
logits at the places asked for, in the order of the entries and of their `want`.
Anything else (a sequence that has started and brings several tokens: a prompt
that comes in pieces; new sequences beside ones that go on) is a *continued
prompt step*: it runs like a prompt step, kernel by kernel, its mixers reading
the earlier positions from the cache (`StepContext.extends`).

Prompt steps with many tokens are cut at sequence borders into pieces of at
most `max_step_tokens`; the pieces are independent, so nothing changes but the
size of the scratch buffers.  Decode steps are replayed from CUDA graphs, one
per (padded batch size, bound on the lengths, mean length in eighths of that
bound); padding rows carry slot -1, touch no cache and change no other row.  Short prompt steps, whose three hundred
launches cost the host more time than the device needs for them, are replayed
from graphs too, one per (padded token count, padded sequence count) once a
shape has come twice; padding tokens form a sequence of their own with slot -1
that stands behind the real ones: it is computed like any other and stored nowhere.

The reference's forward takes one sequence, one offset, and returns the last
position's logits (`qwen/model.go:346-349`, `gemma/gemma.go:196-213`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.cache import CacheError, ModelCache
from ..parts.base import Runtime, StepContext, Workspace
from .model import DecoderModel


class StepError(ValueError):
    """A step that the engine refuses before anything is launched."""


@dataclass
class StepEntry:
    slot: int | None                # None: a padding row of a decode step (touches no cache, changes no other row)
    tokens: Sequence[int]
    want: Sequence[int] = ()        # places among `tokens` whose logits are asked for


def _bucket_batch(n: int) -> int:
    return n if n <= 8 else (n + 7) // 8 * 8


def _bucket_len(n: int) -> int:
    b = 256
    while b < n:
        b *= 2
    return b


_PROMPT_TOKEN_BUCKETS = (16, 32, 48, 64, 96, 128, 192, 256, 320, 384, 448, 512)


def _bucket_prompt_tokens(n: int) -> int:
    for b in _PROMPT_TOKEN_BUCKETS:
        if n <= b:
            return b
    raise ValueError(n)


def _bucket_prompt_seqs(n: int) -> int:
    """Sequences of a graphed prompt step: the real ones and at least one padding sequence."""
    b = 2
    while b < n + 1:
        b *= 2
    return b


def prompt_tables(entries, lens, Tb: int, Tmax: int, Smax: int) -> np.ndarray:
    """The tables of a graphed prompt step, laid out for the largest shape: tokens, positions and sequence
    indices (Tmax each), then slots, lengths before the step (all 0), lengths after it, first rows and wanted rows
    (Smax each).  The tokens from the end of the real ones up to Tb are padding: token 0 at positions 0, 1, ... of
    sequence n_seq, a sequence of its own with slot -1 and their number as its length, so that every row of the
    step is some sequence's and every kernel writes it (it is stored nowhere and no real sequence sees it).  The
    sequences after it have slot -1 and length 0; the first row of each is the end of the one before; wanted
    rows beyond the real ones point at row 0."""
    n_seq, T = len(entries), sum(lens)
    host = np.zeros(3 * Tmax + 5 * Smax, dtype=np.int32)
    first = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    host[0:T] = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
    host[Tmax:Tmax + T] = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    host[Tmax + T:Tmax + Tb] = np.arange(Tb - T, dtype=np.int32)
    host[2 * Tmax:2 * Tmax + T] = np.repeat(np.arange(n_seq, dtype=np.int32), lens)
    host[2 * Tmax + T:2 * Tmax + Tb] = n_seq
    o = 3 * Tmax
    host[o:o + Smax] = -1                            # slots
    host[o:o + n_seq] = [e.slot for e in entries]
    host[o + 2 * Smax:o + 2 * Smax + n_seq] = lens   # lengths after the step
    host[o + 2 * Smax + n_seq] = Tb - T              # the padding tokens' sequence
    host[o + 3 * Smax:o + 4 * Smax] = Tb             # first rows
    host[o + 3 * Smax:o + 3 * Smax + n_seq] = first
    host[o + 3 * Smax + n_seq] = T
    rows = [first[i] + np.asarray(e.want, dtype=np.int32) for i, e in enumerate(entries) if len(e.want)]
    if rows:
        rows = np.concatenate(rows)
        host[o + 4 * Smax:o + 4 * Smax + len(rows)] = rows
    return host


class Stepper:
    MAX_GRAPH_BATCH = 256
    PROMPT_GRAPH_TOKENS = _PROMPT_TOKEN_BUCKETS[-1]     # longer prompt steps keep the device busy past the host
    PROMPT_GRAPH_SEQS = 32                              # padded sequence count of a graphed prompt step, at most
    PROMPT_GRAPHS = 48                                  # graphs kept; the least recently used one goes first

    def __init__(self, model: DecoderModel, cache: ModelCache, rt: Runtime, max_step_tokens: int = 16384,
                 use_graphs: bool = True):
        self.model, self.cache, self.rt = model, cache, rt
        self.ws = Workspace(rt.device)
        self.max_step_tokens = max(1, int(max_step_tokens))
        self.use_graphs = bool(use_graphs) and torch.device(rt.device).type == "cuda" and model.graph_safe
        self._graphs: dict[tuple, tuple] = {}     # (padded batch, length bound, mean length in eighths of it, even) -> graph
        self._prompt_graphs: dict[tuple, tuple] = {}   # (padded tokens, padded sequences, logits wanted) -> (graph,)
        self._prompt_seen: set[tuple] = set()          # shapes that have come once
        self._prompt_meta = None
        self._prompt_logits = None
        self._prompt_stage: list = []
        self._prompt_stage_done: list = []
        self._prompt_stage_next = 0
        self._decode_meta = None
        self._decode_logits = None
        self._stage: list = []
        self._stage_done: list = []
        self._stage_next = 0
        self.h2d_bytes = 0          # bytes of the last decode step's host-to-device copy
        self.launch_counter = 0     # kernels launched by the last decode step (per replay when graphed)

    # ------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], copy: bool = True, tokens_on_device: bool = False):
        """Run one step.  Returns float32 [wanted, vocab] on the device, or None when nothing is wanted.
        With copy=False a decode step returns a view of a buffer that the next step overwrites.
        With tokens_on_device=True a decode step takes its tokens from `token_buffer` as it stands
        (the entries' token values are ignored)."""
        entries = list(entries)
        mode = self._validate(entries)
        if mode == "decode":
            return self._decode(entries, copy, tokens_on_device)
        return self._prefill(entries, extends=mode == "extend")

    def _validate(self, entries) -> str:
        if not entries:
            raise StepError("a step needs at least one sequence")
        seen = set()
        V = self.model.vocab
        fresh = decode = more = 0
        for e in entries:
            if e.slot is None:
                if len(e.tokens) != 1:
                    raise StepError("a padding row brings exactly one token")
                decode += 1
                continue
            if e.slot in seen:
                raise StepError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if not self.cache.is_live(e.slot):
                raise StepError(f"slot {e.slot} is not in use")
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"slot {e.slot}: a sequence must bring at least one token")
            have = self.cache.length(e.slot)
            if have + n > self.cache.max_ctx:
                raise StepError(f"slot {e.slot}: {have} + {n} tokens exceed the context of {self.cache.max_ctx}")
            for t in e.tokens:
                if not 0 <= int(t) < V:
                    raise StepError(f"slot {e.slot}: token id {t} is outside the vocabulary of {V}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {n} tokens")
            if have == 0:
                fresh += 1
            elif n == 1:
                decode += 1
            else:
                more += 1
        if not seen:
            raise StepError("a step of padding rows alone")
        if more or (fresh and decode):
            if len(seen) != len(entries):
                raise StepError("padding rows stand in decode steps only")
            return "extend"
        return "prefill" if fresh else "decode"

    # ------------------------------------------------------------------
    def _prefill(self, entries, extends: bool = False) -> torch.Tensor | None:
        n_want = sum(len(e.want) for e in entries)
        out = torch.empty((n_want, self.model.vocab), dtype=torch.float32, device=self.rt.device) if n_want else None
        pieces, cur, cur_tok = [], [], 0
        for e in entries:
            if cur and cur_tok + len(e.tokens) > self.max_step_tokens:
                pieces.append(cur)
                cur, cur_tok = [], 0
            cur.append(e)
            cur_tok += len(e.tokens)
        pieces.append(cur)
        row0 = 0
        for piece in pieces:
            r = sum(len(e.want) for e in piece)
            self._prefill_piece(piece, out[row0:row0 + r] if r else None, extends)
            row0 += r
        return out

    def _prefill_piece(self, entries, out, extends: bool = False) -> None:
        n_seq = len(entries)
        lens = [len(e.tokens) for e in entries]
        T = sum(lens)
        have = [self.cache.length(e.slot) for e in entries]       # tokens that earlier steps stored
        extends = extends and any(have)
        if self.use_graphs and not extends and T <= self.PROMPT_GRAPH_TOKENS and n_seq < self.PROMPT_GRAPH_SEQS:
            n_want = 0 if out is None else out.shape[0]
            key = (_bucket_prompt_tokens(T), _bucket_prompt_seqs(n_seq), n_want > 0)
            if n_want <= key[1]:
                if key in self._prompt_seen:
                    return self._prefill_graphed(entries, lens, out, key)
                self._prompt_seen.add(key)        # a shape that never comes back is not worth a capture
        first = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        tok_pos = np.concatenate([np.arange(h, h + n, dtype=np.int32) for h, n in zip(have, lens)])
        tok_seq = np.repeat(np.arange(n_seq, dtype=np.int32), lens)
        slots = np.asarray([e.slot for e in entries], dtype=np.int32)
        rows = np.concatenate([first[i] + np.asarray(e.want, dtype=np.int32) for i, e in enumerate(entries)]
                              ).astype(np.int32) if out is not None else np.zeros(0, dtype=np.int32)
        ends = [h + n for h, n in zip(have, lens)]
        for e, n in zip(entries, ends):
            self.cache.reserve(e.slot, n)
        self.cache.sync()
        host = np.concatenate([tokens, tok_pos, tok_seq, slots, np.asarray(have, np.int32),
                               np.asarray(ends, np.int32), first, rows])
        dev = torch.from_numpy(host).to(self.rt.device)
        o = 0

        def take(n):
            nonlocal o
            v = dev[o:o + n]
            o += n
            return v

        ctx = StepContext(rt=self.rt, ws=self.ws, mode="prefill", n_tok=T, n_seq=n_seq, tokens=take(T),
                          tok_pos=take(T), tok_seq=take(T), seq_slot=take(n_seq), seq_start=take(n_seq),
                          seq_end=take(n_seq), seq_first_row=take(n_seq), len_bound=max(ends), extends=extends,
                          step_lens=tuple(lens))
        rows_dev = take(len(rows))
        h = self.model.forward(ctx, self.cache)
        if out is not None:
            self.model.logits(ctx, h, rows_dev, len(rows), out)
        for e, n in zip(entries, ends):
            self.cache.advance(e.slot, n)

    def _prefill_graphed(self, entries, lens, out, key) -> None:
        """A short prompt step through a CUDA graph of its padded shape.  The tables live in one static device
        buffer laid out for the largest shape; padding tokens (token 0) are sequence n_seq, which has slot -1 and
        attends over itself alone, so every row of every buffer of the step is written; the sequences after it
        have slot -1 and length 0; wanted rows beyond the real ones point at row 0 and their logits are dropped."""
        Tb, Sb, wanted = key
        Tmax, Smax = self.PROMPT_GRAPH_TOKENS, self.PROMPT_GRAPH_SEQS
        n_seq, T = len(entries), sum(lens)
        dev = self.rt.device
        if self._prompt_meta is None:
            self._prompt_meta = torch.zeros(3 * Tmax + 5 * Smax, dtype=torch.int32, device=dev)
        if self._prompt_logits is None or self._prompt_logits.shape[0] < Sb:
            self._prompt_graphs.clear()                 # graphs hold the address of the old buffer
            self._prompt_logits = torch.empty((Sb, self.model.vocab), dtype=torch.float32, device=dev)
        n_want = 0 if out is None else out.shape[0]
        host = prompt_tables(entries, lens, Tb, Tmax, Smax)
        o = 3 * Tmax
        for e, n in zip(entries, lens):
            self.cache.reserve(e.slot, n)
        self.cache.sync()
        meta = self._prompt_meta
        self._upload_prompt(host)
        ctx = StepContext(rt=self.rt, ws=self.ws, mode="prefill", n_tok=Tb, n_seq=Sb, tokens=meta[0:Tb],
                          tok_pos=meta[Tmax:Tmax + Tb], tok_seq=meta[2 * Tmax:2 * Tmax + Tb],
                          seq_slot=meta[o:o + Sb], seq_start=meta[o + Smax:o + Smax + Sb],
                          seq_end=meta[o + 2 * Smax:o + 2 * Smax + Sb],
                          seq_first_row=meta[o + 3 * Smax:o + 3 * Smax + Sb], len_bound=Tb)
        rows = meta[o + 4 * Smax:o + 4 * Smax + Sb]
        logits = self._prompt_logits[:Sb]

        def body():
            h = self.model.forward(ctx, self.cache)
            if wanted:
                self.model.logits(ctx, h, rows, Sb, logits)

        hit = self._prompt_graphs.pop(key, None)
        if hit is None:
            body()                                      # once kernel by kernel: every buffer exists afterwards
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            self.ws.begin_capture()
            try:
                with torch.cuda.graph(g):
                    body()
            finally:
                self.ws.end_capture()
            hit = (g,)
            if len(self._prompt_graphs) >= self.PROMPT_GRAPHS:
                self._prompt_graphs.pop(next(iter(self._prompt_graphs)))
        else:
            hit[0].replay()
        self._prompt_graphs[key] = hit                  # most recently used last
        for e, n in zip(entries, lens):
            self.cache.advance(e.slot, n)
        if n_want:
            out.copy_(logits[:n_want])

    def _upload_prompt(self, host: np.ndarray) -> None:
        """Host tables of a graphed prompt step -> the static device tables, through pinned staging buffers."""
        if not self._prompt_stage:
            self._prompt_stage = [torch.empty(host.shape[0], dtype=torch.int32).pin_memory() for _ in range(4)]
            self._prompt_stage_done = [None] * len(self._prompt_stage)
        i = self._prompt_stage_next
        self._prompt_stage_next = (i + 1) % len(self._prompt_stage)
        if self._prompt_stage_done[i] is not None:
            self._prompt_stage_done[i].synchronize()
        self._prompt_stage[i].numpy()[...] = host
        self._prompt_meta.copy_(self._prompt_stage[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._prompt_stage_done[i] = ev

    # ------------------------------------------------------------------
    def _decode(self, entries, copy: bool, tokens_on_device: bool = False) -> torch.Tensor | None:
        n_seq = len(entries)
        B = _bucket_batch(n_seq)
        pos = [self.cache.length(e.slot) if e.slot is not None else 0 for e in entries]
        for e, p in zip(entries, pos):
            if e.slot is not None:
                self.cache.reserve(e.slot, p + 1)
        self.cache.sync()
        bound = _bucket_len(max(pos) + 1)
        # how full the batch is: the mean length over its rows (padding rows count as empty) in eighths of the bound.
        # A launch shape that suits eight sequences at the bound wastes most of the GPU on sixty-four of which one
        # is; the eighth is part of a recorded step's key, so a shape is replayed only for batches like its own.
        fill = max(1, min(8, -(-8 * (sum(pos) + n_seq) // (B * bound))))
        real = [p + 1 for e, p in zip(entries, pos) if e.slot is not None]
        even = B == n_seq and 4 * min(real) >= 3 * max(real)
        graphs = self.use_graphs and B <= self.MAX_GRAPH_BATCH
        dev = self.rt.device
        if self._decode_meta is None:
            self._decode_meta = torch.zeros((7, self.MAX_GRAPH_BATCH), dtype=torch.int32, device=dev)
        if self._decode_logits is None or self._decode_logits.shape[0] < B:
            self._graphs.clear()        # graphs hold the address of the old buffer
            self._decode_logits = torch.empty((max(B, 8), self.model.vocab), dtype=torch.float32, device=dev)
        width = self.MAX_GRAPH_BATCH if B <= self.MAX_GRAPH_BATCH else B
        host = np.zeros((7, width), dtype=np.int32)
        host[0, :n_seq] = [int(e.tokens[0]) for e in entries]
        host[1, :n_seq] = pos
        host[2, :B] = np.arange(B)
        host[3, :] = -1
        host[3, :n_seq] = [e.slot if e.slot is not None else -1 for e in entries]
        host[4, :n_seq] = pos
        host[5, :B] = 1
        host[5, :n_seq] = np.asarray(pos) + 1
        host[6, :B] = np.arange(B)
        if B <= self.MAX_GRAPH_BATCH:
            meta = self._decode_meta
            self._upload(host, meta, skip_tokens=tokens_on_device)
        else:
            meta = torch.from_numpy(host).to(dev)
        ctx = StepContext(rt=self.rt, ws=self.ws, mode="decode", n_tok=B, n_seq=B, tokens=meta[0, :B],
                          tok_pos=meta[1, :B], tok_seq=meta[2, :B], seq_slot=meta[3, :B], seq_start=meta[4, :B],
                          seq_end=meta[5, :B], seq_first_row=meta[6, :B], len_bound=bound,
                          len_mean=-(-fill * bound // 8), len_even=even)
        logits = self._decode_logits[:B]
        key = (B, bound, fill, even)
        if graphs and key in self._graphs:
            g, n_launch = self._graphs[key]
            g.replay()
            self.launch_counter = n_launch
        else:
            before = self.rt.ops.launch_count() if hasattr(self.rt.ops, "launch_count") else 0
            self._decode_body(ctx, logits)
            n_launch = (self.rt.ops.launch_count() if hasattr(self.rt.ops, "launch_count") else 0) - before
            self.launch_counter = n_launch
            if graphs:
                self._graphs[key] = (self._capture(ctx, logits), n_launch)
        for e, p in zip(entries, pos):
            if e.slot is not None:
                self.cache.advance(e.slot, p + 1)
        wanted = [i for i, e in enumerate(entries) if len(e.want)]
        if not wanted:
            return None
        if len(wanted) == n_seq:
            res = logits[:n_seq]
        else:
            res = logits.index_select(0, torch.tensor(wanted, dtype=torch.long, device=dev))
            copy = False
        return res.clone() if copy else res

    def token_buffer(self, n: int) -> torch.Tensor:
        """The device buffer that a decode step reads its tokens from (int32 [n]).  A sampler that
        writes the next tokens here feeds them to the next step without a trip to the host
        (`step(..., tokens_on_device=True)`); the reference's greedy loop keeps the token on the
        device in the same way (`qwen/model.go:354-404`)."""
        if n > self.MAX_GRAPH_BATCH:
            raise StepError(f"device-fed tokens are limited to {self.MAX_GRAPH_BATCH} sequences")
        if self._decode_meta is None:
            self._decode_meta = torch.zeros((7, self.MAX_GRAPH_BATCH), dtype=torch.int32, device=self.rt.device)
        return self._decode_meta[0, :n]

    def _upload(self, host: np.ndarray, meta: torch.Tensor, skip_tokens: bool) -> None:
        """Host tables of a decode step -> the static device tables, through pinned staging buffers.
        A staging buffer is reused only after the copy that read it has run."""
        if torch.device(self.rt.device).type != "cuda":
            (meta[1:] if skip_tokens else meta).copy_(torch.from_numpy(host[1:] if skip_tokens else host))
            return
        if not self._stage:
            self._stage = [torch.empty((7, self.MAX_GRAPH_BATCH), dtype=torch.int32).pin_memory() for _ in range(4)]
            self._stage_done = [None] * len(self._stage)
        i = self._stage_next
        self._stage_next = (i + 1) % len(self._stage)
        if self._stage_done[i] is not None:
            self._stage_done[i].synchronize()
        self._stage[i].numpy()[...] = host
        if skip_tokens:
            meta[1:].copy_(self._stage[i][1:], non_blocking=True)
        else:
            meta.copy_(self._stage[i], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_done[i] = ev
        self.h2d_bytes = (6 if skip_tokens else 7) * self.MAX_GRAPH_BATCH * 4

    def _decode_body(self, ctx: StepContext, logits: torch.Tensor) -> None:
        h = self.model.forward(ctx, self.cache)
        self.model.logits(ctx, h, None, ctx.n_tok, logits)

    def _capture(self, ctx: StepContext, logits: torch.Tensor):
        """Record the decode step that has just run once (all its buffers exist) into a graph."""
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        self.ws.begin_capture()
        try:
            with torch.cuda.graph(g):
                self._decode_body(ctx, logits)
        finally:
            self.ws.end_capture()
        return g
