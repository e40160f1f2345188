"""The generation loop: requests in, replies out, batch after batch.

The loop makes decisions only; the model, the cache and the sampler are behind
a small backend interface, so the loop can be tested with a fake one:

    backend.max_batch, backend.max_context
    backend.fits(final_lengths) -> bool          room for sequences of these lengths together
    backend.open() -> handle                      a sequence's place in the cache
    backend.close(handle)
    backend.prefill(handles, prompts, request_ids, banned) -> first tokens
    backend.decode_start(handles, last_tokens, request_ids, token_index, replies) -> ticket
    backend.decode_finish(ticket) -> next tokens
    backend.lookahead                              whether a step may start before the one before it is read
    backend.keeps_layout(n_live, n_rows) -> bool  whether n_live sequences may stay in a layout of n_rows rows

One batch: the prompts start together in one prompt step and get their first
token each; then decode steps over the sequences still alive.  A stop token ends
a reply and is not part of it; a reply also ends at `max_tokens` (one limit, or one per request) or when the
context is full; a sequence that has ended leaves the batch and gives its place
back at once.  Requests that do not fit into one batch are served in as many
batches as it takes, in the order given.

With `backend.lookahead` the loop starts step k+1 before it has read the tokens of
step k: the backend feeds step k's tokens to step k+1 on the device (`last_tokens`
is then None), so the device never waits for the host.  Rows keep their place in the
layout meanwhile; a row whose reply has ended becomes a hole (handle None).  Ends by
length are known beforehand and cost nothing; a stop token is seen one step late, and
the one token computed past it is dropped.  When enough rows are holes the loop lets
the pipeline drain and forms a tighter layout from the tokens it holds.

From the reference's loop (`qwen/session.go:363-484`, `qwen/model.go:170-212`):
prefill, sample, then {stop? -> end; append; OnToken; length? -> end; cancel? ->
end; forward one token; sample}; default of 512 tokens (`engine.go:312-315`);
the optional masking of stop tokens at the first position (`qwen/session.go:377-391`);
its greedy loop likewise keeps the token on the device (`qwen/model.go:354-404`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Iterable, Sequence

DEFAULT_MAX_TOKENS = 512


class GenerationError(ValueError):
    pass


@dataclass
class Reply:
    tokens: list[int] = field(default_factory=list)
    finish_reason: str = ""       # "stop", "length", "cancel", "empty"


def plan_batches(final_lengths: Sequence[int], max_batch: int, fits: Callable[[Sequence[int]], bool]) -> list[list[int]]:
    """Cut request indices 0..n-1, in order, into batches that fit."""
    batches, cur = [], []
    for i, n in enumerate(final_lengths):
        if not fits([n]):
            raise GenerationError(f"request {i} needs room for {n} tokens, more than the cache holds at all")
        if cur and (len(cur) >= max_batch or not fits([final_lengths[j] for j in cur] + [n])):
            batches.append(cur)
            cur = []
        cur.append(i)
    if cur:
        batches.append(cur)
    return batches


def generate(backend, prompts: Sequence[Sequence[int]], max_tokens: int = DEFAULT_MAX_TOKENS,
             stop: Iterable[int] = (), on_token: Callable[[int, int], None] | None = None,
             cancel: Callable[[], bool] | None = None, mask_stop_on_first: bool = False) -> list[Reply]:
    # one limit for every request, or one per request; <= 0 means the default
    if isinstance(max_tokens, (list, tuple)):
        if len(max_tokens) != len(prompts):
            raise GenerationError(f"{len(max_tokens)} token limits for {len(prompts)} requests")
        limits = [int(m) if int(m) > 0 else DEFAULT_MAX_TOKENS for m in max_tokens]
    else:
        limits = [int(max_tokens) if int(max_tokens) > 0 else DEFAULT_MAX_TOKENS] * len(prompts)
    stop = frozenset(int(s) for s in stop)
    replies = [Reply() for _ in prompts]
    todo = []
    for i, p in enumerate(prompts):
        if len(p) == 0:                       # the reference returns nothing for an empty prompt
            replies[i].finish_reason = "empty"
        elif len(p) >= backend.max_context:
            raise GenerationError(f"request {i}: a prompt of {len(p)} tokens leaves no room in a context of "
                                  f"{backend.max_context}")
        else:
            todo.append(i)
    final = [min(len(prompts[i]) + limits[i], backend.max_context) for i in todo]
    cancelled = False
    for batch in plan_batches(final, backend.max_batch, backend.fits):
        ids = [todo[j] for j in batch]
        if cancelled:
            for i in ids:
                replies[i].finish_reason = "cancel"
            continue
        cancelled = _Batch(backend, ids, prompts, replies, limits, stop, on_token, cancel, mask_stop_on_first).run()
    return replies


class _Batch:
    def __init__(self, backend, ids, prompts, replies, max_tokens, stop, on_token, cancel, mask_stop_on_first):
        self.b, self.ids, self.prompts, self.replies = backend, ids, prompts, replies
        self.max_tokens, self.stop, self.on_token, self.cancel = max_tokens, stop, on_token, cancel
        self.mask_stop_on_first = mask_stop_on_first
        self.handles: dict[int, object] = {}

    def _full_after(self, i: int, more: int) -> bool:
        """Whether reply i is at its length once `more` further tokens have been added."""
        n = len(self.replies[i].tokens) + more
        return n >= self.max_tokens[i] or len(self.prompts[i]) + n >= self.b.max_context

    def _take(self, rows, toks) -> None:
        """The tokens of one step: append or end, in row order; holes and ended replies are skipped."""
        for i, tok in zip(rows, toks):
            if i is None or self.replies[i].finish_reason:
                continue
            r, tok = self.replies[i], int(tok)
            if tok in self.stop:
                r.finish_reason = "stop"
            else:
                r.tokens.append(tok)
                if self.on_token is not None:
                    self.on_token(i, tok)
                if self._full_after(i, 0):
                    r.finish_reason = "length"
            if r.finish_reason:
                self.b.close(self.handles.pop(i))

    def _start(self, rows, from_device: bool):
        live = [i is not None for i in rows]
        return self.b.decode_start(
            [self.handles[i] if ok else None for i, ok in zip(rows, live)],
            None if from_device else [self.replies[i].tokens[-1] if ok else 0 for i, ok in zip(rows, live)],
            rows,
            [len(self.replies[i].tokens) + (1 if from_device else 0) if ok else 0 for i, ok in zip(rows, live)],
            [self.replies[i].tokens if ok else () for i, ok in zip(rows, live)])

    def run(self) -> bool:
        """True when the caller cancelled."""
        b = self.b
        try:
            for i in self.ids:
                self.handles[i] = b.open()
            banned = sorted(self.stop) if (self.mask_stop_on_first and self.stop) else None
            toks = b.prefill([self.handles[i] for i in self.ids], [list(self.prompts[i]) for i in self.ids], self.ids,
                             banned)
            self._take(self.ids, toks)
            rows, pending = [], None
            asked_to_stop = lambda: self.cancel is not None and self.cancel()     # asked before every step's start
            while True:
                if pending is None:                               # form a layout from the replies still open
                    rows = [i for i in self.ids if not self.replies[i].finish_reason]
                    if not rows:
                        return False
                    if asked_to_stop():
                        return self._cancel_all()
                    pending = self._start(rows, from_device=False)
                nxt, nxt_rows, stop_now = None, None, False
                if getattr(b, "lookahead", False):
                    # rows that are still open after the pending step, as far as that can be known now
                    nxt_rows = [i if (i is not None and not self.replies[i].finish_reason and not self._full_after(i, 1))
                                else None for i in rows]
                    n_live = sum(i is not None for i in nxt_rows)
                    if n_live and b.keeps_layout(n_live, len(rows)):
                        stop_now = asked_to_stop()
                        if not stop_now:
                            nxt = self._start(nxt_rows, from_device=True)
                self._take(rows, b.decode_finish(pending))
                if stop_now:
                    return self._cancel_all()
                rows, pending = (nxt_rows, nxt) if nxt is not None else (rows, None)
                # rows of `nxt` whose reply met a stop token in the step just read are skipped by _take
        finally:
            for h in self.handles.values():
                b.close(h)
            self.handles.clear()

    def _cancel_all(self) -> bool:
        for i in self.ids:
            if not self.replies[i].finish_reason:
                self.replies[i].finish_reason = "cancel"
        return True
