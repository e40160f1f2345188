"""Helpers shared by the engine tests: building an engine on the GPU kernels or, for
the host-side tests, on the plain kernel statements; driving steps; comparing logits."""
from __future__ import annotations

import torch

from tests.conftest import BF16_MODEL_TOL, F32_MODEL_TOL


def make_engine(model_dir: str, dtype, on: str = "cuda", **kw):
    """on='cuda': the product path.  on='refs': the same engine over tests/kernel_refs.py on the CPU."""
    import janis_b200
    if on == "cuda":
        return janis_b200.open(model_dir, dtype=dtype, **kw)
    from janis_b200.config.base import read_config_json
    from janis_b200.engine.engine import Engine, _dtype, build_model
    from janis_b200.parts.base import Runtime, WeightStore
    from janis_b200.weights.loader import load_tensors
    from tests import kernel_refs
    _, cfg, model = build_model(read_config_json(model_dir))
    rt = Runtime(_dtype(dtype), "cpu", kernel_refs)
    model.load(WeightStore(load_tensors(model_dir, model.tensor_specs(), "cpu", model.ignorable_tensors)), rt)
    kw.pop("device", None)
    kw.setdefault("use_graphs", False)
    return Engine(model, rt, kw.pop("max_tokens", 8192), kw.pop("max_batch", None), kw.pop("max_context", None),
                  kw.pop("max_step_tokens", 16384), kw.pop("use_graphs"))


def model_tol(dtype) -> float:
    return F32_MODEL_TOL if dtype in ("float32", torch.float32) else BF16_MODEL_TOL


def assert_logits(got: torch.Tensor, want: torch.Tensor, dtype, what: str) -> None:
    got, want = got.detach().double().cpu(), want.double()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = want.abs().max().item()
    err = (got - want).abs()
    worst = err.max().item()
    if worst > model_tol(dtype) * scale:
        row = int(err.max(dim=1).values.argmax())
        first_bad = int((err.max(dim=1).values > model_tol(dtype) * scale).nonzero()[0])
        raise AssertionError(f"{what}: max err {worst:.3e} > {model_tol(dtype):.0e} x scale {scale:.3e}; "
                             f"worst row {row}, first row over tolerance {first_bad} of {got.shape[0]}")


def run_requests(engine, requests, prompt_lens, max_live=None):
    """Feed `requests` (lists of token ids) through engine.step in batches that start together:
    request i brings its first prompt_lens[i] tokens in the prompt step, then one token per step;
    requests that run out leave the batch and free their slot.  Batches follow one another,
    `max_live` requests each, so slots and pages are used again.  Returns the logits at every
    position of every request: list of [len_i, vocab] tensors (on the CPU)."""
    from janis_b200 import StepEntry
    n = len(requests)
    max_live = max_live or n
    got = [[] for _ in range(n)]
    for b0 in range(0, n, max_live):
        ids = list(range(b0, min(n, b0 + max_live)))
        slots = {i: engine.alloc_slot() for i in ids}
        out = engine.step([StepEntry(slots[i], requests[i][:prompt_lens[i]], list(range(prompt_lens[i]))) for i in ids])
        o = 0
        for i in ids:
            got[i].append(out[o:o + prompt_lens[i]].cpu())
            o += prompt_lens[i]
        pos = {i: prompt_lens[i] for i in ids}
        live = [i for i in ids]
        while True:
            for i in list(live):
                if pos[i] >= len(requests[i]):
                    live.remove(i)
                    engine.free_slot(slots.pop(i))
            if not live:
                break
            out = engine.step([StepEntry(slots[i], [requests[i][pos[i]]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1].cpu())
                pos[i] += 1
        engine.cache.audit()
    return [torch.cat(g) for g in got]


def run_in_pieces(engine, requests, chunk):
    """Feed each request in steps of `chunk` tokens onto what the steps before left in the cache, the requests
    side by side (a shorter one ends earlier); logits at every position: list of [len_i, vocab] tensors (CPU)."""
    from janis_b200 import StepEntry
    slots = [engine.alloc_slot() for _ in requests]
    got = [[] for _ in requests]
    pos = [0] * len(requests)
    while any(p < len(r) for p, r in zip(pos, requests)):
        live = [i for i, r in enumerate(requests) if pos[i] < len(r)]
        take = [min(chunk, len(requests[i]) - pos[i]) for i in live]
        out = engine.step([StepEntry(slots[i], requests[i][pos[i]:pos[i] + t], list(range(t))) for i, t in zip(live, take)])
        o = 0
        for i, t in zip(live, take):
            got[i].append(out[o:o + t].cpu())
            o += t
            pos[i] += t
    for s in slots:
        engine.free_slot(s)
    engine.cache.audit()
    return [torch.cat(g) for g in got]
