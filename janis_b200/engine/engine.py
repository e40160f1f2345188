"""The Python entry point: open a model folder, generate, close.

In the manner of the reference's Go module: `llm.Open(dir)` loads config, then
weights, then the model chosen by the configuration (`engine.go:131-237`);
`Engine.Chat(msgs, Options{Temp, TopP, MaxTokens, Seed, Cancel, OnToken})`
generates (`engine.go:57-87`, `:288-423`); `Close` frees (`engine.go:464`).
This library works on token ids (tokenizer and chat templates are not part of
it), so `generate` takes prompts as lists of ids and returns lists of ids.
"""
from __future__ import annotations

import os
from typing import Callable, Iterable, Sequence

import torch

from ..cache.cache import ModelCache
from ..config.base import ConfigError, read_config_json
from ..kernels import ops as cuda_ops
from ..parts.base import Runtime, WeightStore
from ..registry import resolve
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import load_tensors, random_tensors, write_model_folder
from . import generate as loop
from .step import StepEntry, Stepper

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    try:
        return _DTYPES[d]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', found {d!r}") from None


class Engine:
    """A loaded model with its cache, step function and sampler."""

    def __init__(self, model, rt: Runtime, max_tokens: int, max_batch: int | None = None,
                 max_context: int | None = None, max_step_tokens: int = 16384, use_graphs: bool = True):
        self.model = model
        self.config = model.config
        self.rt = rt
        self.max_context = int(max_context or model.max_context)
        self.cache = ModelCache(model.cache_line_needs(), max_tokens, self.max_context, rt.dtype, rt.device,
                                max_seqs=max_batch)
        self.max_batch = self.cache.n_slots
        self.stepper = Stepper(model, self.cache, rt, max_step_tokens, use_graphs)
        self.sampler = Sampler(rt)
        self.stop_tokens = tuple(model.stop_tokens)
        self._closed = False
        # counters of bounded device waits that gave up: read wherever the host waits for the device anyway
        watch = getattr(rt.ops, "WaitWatch", None)
        self.watch = watch() if watch is not None and torch.device(rt.device).type == "cuda" else None
        if self.watch is not None:
            self.check_health(quiet=True)        # what happened before this engine existed is not its business

    # -- the step function, for callers that drive it themselves ----------------
    def alloc_slot(self) -> int:
        return self.cache.alloc_slot()

    def free_slot(self, slot: int) -> None:
        self.cache.free_slot(slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor | None:
        """See `Stepper.step`: float32 logits [wanted, vocab] on the device."""
        return self.stepper.step(entries)

    def check_health(self, quiet: bool = False) -> None:
        """Waits for the device and raises `KernelError` if a kernel gave up one of its bounded waits since the
        last check (a CTA that gives up returns without its result, so the steps in between are not to be
        trusted).  `generate` does this by itself wherever it reads tokens; a caller that drives `step` calls it
        when it reads logits."""
        if self.watch is None:
            return
        self.watch.request()
        torch.cuda.current_stream().synchronize()
        self.watch.check(quiet)

    # -- generation ---------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], temp: float = 0.0, top_p: float = 1.0,
                 max_tokens: int = loop.DEFAULT_MAX_TOKENS, seed: int = 0, stop: Iterable[int] | None = None,
                 on_token: Callable[[int, int], None] | None = None, cancel: Callable[[], bool] | None = None,
                 repeat_penalty: float = 1.0, repeat_last_n: int = 64, mask_stop_on_first: bool = False,
                 return_replies: bool = False, *, temperature: float | None = None,
                 max_new_tokens: int | None = None, stop_tokens: Iterable[int] | None = None):
        """Replies (lists of token ids) to prompts (lists of token ids), in order.

        temp <= 0 is greedy; top_p outside (0, 1] means 1; max_tokens is one limit for every reply or a list
        with one per request, <= 0 means 512; `stop` defaults to
        the model's end-of-sequence ids and a stop token is not part of the reply; `on_token(request,
        token)` hears every token as it is produced; `cancel()` is asked before every decode step.
        With return_replies=True the result is a list of `Reply` (tokens and finish_reason).
        `temperature`, `max_new_tokens` and `stop_tokens` are other names of temp, max_tokens and stop."""
        if self._closed:
            raise RuntimeError("the engine is closed")
        temp = temp if temperature is None else temperature
        max_tokens = max_tokens if max_new_tokens is None else max_new_tokens
        stop = stop if stop_tokens is None else stop_tokens
        params = SamplingParams(temp, top_p, seed, repeat_penalty, repeat_last_n).normalized()
        backend = _Backend(self, params)
        replies = loop.generate(backend, prompts, max_tokens, self.stop_tokens if stop is None else stop,
                                on_token, cancel, mask_stop_on_first)
        return replies if return_replies else [r.tokens for r in replies]

    def close(self) -> None:
        """Drop the model, the cache and the graphs (`engine.go:464-475`)."""
        self._closed = True
        self.stepper = None
        self.cache = None
        self.model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


class _Backend:
    """What the generation loop needs, on top of the engine's step function and sampler.

    A decode step is started and read in two calls.  The chosen tokens are written into the step
    function's device token buffer, from where the next step can take them without the host
    (`last_tokens=None`), and copied to pinned host memory behind an event, so that reading step k
    does not wait for step k+1, which may already be queued."""

    def __init__(self, engine: Engine, params: SamplingParams):
        self.e = engine
        self.params = params
        self.max_batch = engine.max_batch
        self.max_context = engine.max_context
        on_gpu = torch.device(engine.rt.device).type == "cuda"
        # the repetition penalty needs the reply so far on the host before the next token is picked
        self.lookahead = on_gpu and not params.repeat_penalty > 1.0
        self._pinned = [torch.empty((Stepper.MAX_GRAPH_BATCH,), dtype=torch.int32).pin_memory() for _ in range(4)] \
            if on_gpu else None
        self._turn = 0

    def fits(self, final_lengths) -> bool:
        return self.e.cache.can_hold(final_lengths)

    def keeps_layout(self, n_live: int, n_rows: int) -> bool:
        """Holes are cheap while they do not push the step into a larger padded batch than it needs."""
        from .step import _bucket_batch
        return n_rows <= Stepper.MAX_GRAPH_BATCH and _bucket_batch(n_live) == _bucket_batch(n_rows)

    def open(self) -> int:
        return self.e.cache.alloc_slot()

    def close(self, handle: int) -> None:
        self.e.cache.free_slot(handle)

    def prefill(self, handles, prompts, request_ids, banned):
        entries = [StepEntry(h, p, (len(p) - 1,)) for h, p in zip(handles, prompts)]
        logits = self.e.stepper.step(entries, copy=False)
        toks = self.e.sampler.sample(logits, self.params, request_ids, [0] * len(handles), None, banned)
        watch = self.e.watch
        if watch is not None:
            watch.request()
        toks = toks.tolist()          # waits for the stream: the counters of given-up waits have arrived too
        if watch is not None:
            watch.check()
        return toks

    def decode_start(self, handles, last_tokens, request_ids, token_index, replies):
        n = len(handles)
        st = self.e.stepper
        entries = [StepEntry(h, ((last_tokens[i] if last_tokens is not None else 0),), (0,))
                   for i, h in enumerate(handles)]
        logits = st.step(entries, copy=False, tokens_on_device=last_tokens is None)
        ids = [r if r is not None else 0 for r in request_ids]
        watch = self.e.watch
        if n > Stepper.MAX_GRAPH_BATCH or self._pinned is None:
            toks = self.e.sampler.sample(logits, self.params, ids, token_index, replies)
            if watch is not None:
                watch.request()
            return toks
        out = st.token_buffer(n)
        self.e.sampler.sample(logits, self.params, ids, token_index, replies, out=out)
        host = self._pinned[self._turn % len(self._pinned)]
        self._turn += 1
        host[:n].copy_(out, non_blocking=True)
        if watch is not None:
            watch.request()           # the counters of given-up waits travel with the tokens
        done = torch.cuda.Event()
        done.record()
        return (host, done, n)

    def decode_finish(self, ticket):
        watch = self.e.watch
        if isinstance(ticket, torch.Tensor):
            toks = ticket.tolist()
        else:
            host, done, n = ticket
            done.synchronize()        # the one wait of a step: n token ids
            toks = host[:n].tolist()
        if watch is not None:
            watch.check()
        return toks


# ---------------------------------------------------------------------------
# opening
# ---------------------------------------------------------------------------

def _runtime(dtype, device) -> Runtime:
    if not torch.cuda.is_available():
        raise RuntimeError("janis_b200 needs a CUDA device (sm_100a); none is visible and there is no "
                           "CPU implementation")
    return Runtime(_dtype(dtype), device, cuda_ops)


def build_model(raw_config: dict, where: str = "config.json"):
    """(architecture, typed configuration, model of parts) that a parsed config.json describes."""
    arch = resolve(raw_config, where)
    cfg = arch.config_class.from_dict(raw_config, where)
    return arch, cfg, arch.build(cfg)


def open(model_dir: str, dtype="bfloat16", max_tokens: int = 8192, max_batch: int | None = None,
         max_context: int | None = None, device="cuda:0", use_graphs: bool = True,
         max_step_tokens: int = 16384) -> Engine:
    """Load config.json and the safetensors of `model_dir` and build the engine.

    `max_tokens` is how many tokens the cache holds over all live sequences (each
    sequence's count rounded up to whole pages of 64); `max_batch` bounds the sequences
    alive at once (default: as many as there are pages)."""
    raw = read_config_json(model_dir)
    _, cfg, model = build_model(raw, os.path.join(model_dir, "config.json"))
    rt = _runtime(dtype, device)
    store = WeightStore(load_tensors(model_dir, model.tensor_specs(), rt.device, model.ignorable_tensors))
    model.load(store, rt)         # parts that fuse tensors give the stored ones up as they go
    del store
    return Engine(model, rt, max_tokens, max_batch, max_context, max_step_tokens, use_graphs)


load = open     # the same call under the name that Python libraries usually give it


def from_config(raw_config: dict, seed: int = 0, dtype="bfloat16", max_tokens: int = 8192,
                max_batch: int | None = None, max_context: int | None = None, device="cuda:0",
                use_graphs: bool = True, max_step_tokens: int = 16384) -> Engine:
    """An engine with random weights drawn on the device from (seed, tensor name): no folder is written."""
    _, cfg, model = build_model(raw_config, "config")
    rt = _runtime(dtype, device)
    store = WeightStore(random_tensors(model.tensor_specs(), seed, rt.device))
    model.load(store, rt)
    del store
    return Engine(model, rt, max_tokens, max_batch, max_context, max_step_tokens, use_graphs)


def write_random_model(model_dir: str, raw_config: dict, seed: int = 0, dtype="bfloat16") -> None:
    """Write config.json and model.safetensors with random weights drawn from (seed, tensor name):
    matrices and the embedding N(0, 0.02), norm weights N(0, 0.1)."""
    _, cfg, model = build_model(raw_config, "config")
    tensors = random_tensors(model.tensor_specs(), seed, "cpu", _dtype(dtype))
    write_model_folder(model_dir, cfg.to_dict(), tensors, {"format": "pt", "seed": str(seed)})
