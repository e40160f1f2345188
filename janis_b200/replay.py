"""Trace replay: feed given token ids through a model step by step and write logits.

It samples nothing and has no model code of its own: it drives the engine's step
function, cache and kernels, the ones generation uses.  Input is one JSON object
per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` gives each request's next tokens and the places among them whose logits
are wanted; a request gets a cache slot when it first appears.  The usual trace
has steps whose requests either all start or all go on by one token; a request
that has started may also bring several tokens (a prompt that comes in pieces),
beside others that start or go on.  `end` names requests that are
finished after the step: their slots are given back.  For a step in which
something is wanted, `<out>/<step>.f32` receives the logits, little-endian
float32 [wanted, vocab], in the order of the entries and of `want`.  After every
step a line `done <step>` is printed and flushed.

The reference's counterpart prints the five highest logits and the greedy ids
for ids given on the command line (`cmd/llmoracle/main.go:26-98`).
"""
from __future__ import annotations

import json
import os
import sys
from typing import Iterable, TextIO

import numpy as np

from .engine.step import StepEntry


class TraceError(ValueError):
    pass


def run_trace(engine, lines: Iterable[str], out_dir: str, report: TextIO = sys.stdout) -> int:
    """Replay the steps in `lines`; returns the number of steps run."""
    os.makedirs(out_dir, exist_ok=True)
    slots: dict[str, int] = {}
    n = 0
    for lineno, line in enumerate(lines, 1):
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
            step = rec["step"]
            entries = rec["entries"]
            ended = rec.get("end", []) or []
        except (json.JSONDecodeError, KeyError, TypeError) as e:
            raise TraceError(f"input line {lineno}: not a step record: {e}") from e
        batch = []
        for ent in entries:
            rid = str(ent["id"])
            if rid not in slots:
                slots[rid] = engine.alloc_slot()
            batch.append(StepEntry(slots[rid], [int(t) for t in ent["tokens"]],
                                   [int(w) for w in ent.get("want", []) or []]))
        if batch:
            logits = engine.step(batch)
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
            if hasattr(engine, "check_health"):
                engine.check_health()     # a kernel that gave up a bounded wait: no logits of this run are to be trusted
        for rid in ended:
            rid = str(rid)
            if rid not in slots:
                raise TraceError(f"input line {lineno}: request {rid!r} ends but never started")
            engine.free_slot(slots.pop(rid))
        n += 1
        print(f"done {step}", file=report, flush=True)
    return n


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64); sizes the cache")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    args = ap.parse_args(argv)
    from .engine import engine as eng_mod
    from .config.base import read_config_json
    raw = read_config_json(args.model)
    max_tokens = max(64, args.max_tokens)
    ctx = max(int(raw.get("max_position_embeddings", 0) or 0), (max_tokens + 63) // 64 * 64)
    engine = eng_mod.open(args.model, dtype=args.dtype, max_tokens=max_tokens, max_context=ctx,
                          use_graphs=not args.no_graphs)
    try:
        run_trace(engine, iter(sys.stdin.readline, ""), args.out)
    finally:
        engine.close()
    return 0
