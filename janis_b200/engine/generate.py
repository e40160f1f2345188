"""The generation loop: requests in, replies out, batch after batch.

The loop makes decisions only; the model, the cache and the sampler are behind
a small backend interface, so the loop can be tested with a fake one:

    backend.max_batch, backend.max_context
    backend.fits(final_lengths) -> bool         room for sequences of these lengths together
    backend.open() -> handle                     a sequence's place in the cache
    backend.close(handle)
    backend.prefill(handles, prompts, request_ids, banned) -> first tokens
    backend.decode(handles, last_tokens, request_ids, token_index, replies) -> next tokens

One batch: the prompts start together in one prompt step and get their first
token each; then decode steps over the sequences still alive.  A stop token ends
a reply and is not part of it; a reply also ends at `max_tokens` or when the
context is full; a sequence that has ended leaves the batch and gives its place
back at once.  Requests that do not fit into one batch are served in as many
batches as it takes, in the order given.

From the reference's loop (`qwen/session.go:363-484`, `qwen/model.go:170-212`):
prefill, sample, then {stop? -> end; append; OnToken; length? -> end; cancel? ->
end; forward one token; sample}; default of 512 tokens (`engine.go:312-315`);
the optional masking of stop tokens at the first position (`qwen/session.go:377-391`).
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
    if max_tokens <= 0:
        max_tokens = DEFAULT_MAX_TOKENS
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
    final = [min(len(prompts[i]) + max_tokens, backend.max_context) for i in todo]
    cancelled = False
    for batch in plan_batches(final, backend.max_batch, backend.fits):
        ids = [todo[j] for j in batch]
        if cancelled:
            for i in ids:
                replies[i].finish_reason = "cancel"
            continue
        cancelled = _run_batch(backend, ids, prompts, replies, max_tokens, stop, on_token, cancel,
                               mask_stop_on_first)
    return replies


def _run_batch(backend, ids, prompts, replies, max_tokens, stop, on_token, cancel, mask_stop_on_first) -> bool:
    handles = {}
    try:
        for i in ids:
            handles[i] = backend.open()
        banned = sorted(stop) if (mask_stop_on_first and stop) else None
        toks = backend.prefill([handles[i] for i in ids], [list(prompts[i]) for i in ids], ids, banned)
        live = list(ids)
        while True:
            nxt = []
            for i, tok in zip(live, toks):
                tok = int(tok)
                r = replies[i]
                if tok in stop:
                    r.finish_reason = "stop"
                else:
                    r.tokens.append(tok)
                    if on_token is not None:
                        on_token(i, tok)
                    if len(r.tokens) >= max_tokens or len(prompts[i]) + len(r.tokens) >= backend.max_context:
                        r.finish_reason = "length"
                if r.finish_reason:
                    backend.close(handles.pop(i))
                else:
                    nxt.append(i)
            live = nxt
            if not live:
                return False
            if cancel is not None and cancel():
                for i in live:
                    replies[i].finish_reason = "cancel"
                return True
            toks = backend.decode([handles[i] for i in live], [replies[i].tokens[-1] for i in live], live,
                                  [len(replies[i].tokens) for i in live], [replies[i].tokens for i in live])
    finally:
        for h in handles.values():
            backend.close(h)
