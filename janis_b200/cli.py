"""The `janis` command line.

In the manner of the reference's: a verb first, then flags; an unknown or missing
verb prints the usage and exits with 2 (`cmd/janis/main.go:27-58`).  The reference's
verbs serve and manage its HTTP server, which this library does not have; the
verbs here are the ones of its small runners: one generation from a loaded model
(`cmd/llmsmoke/main.go:22-75`), replay of given ids (`cmd/llmoracle/main.go:26-98`)
and a benchmark (`cmd/enginebench/main.go:56-64`).  Option names are the
reference's request fields: temp, top-p, max-tokens, seed (`engine.go:57-87`,
`serve/serve.go:272-276`).  Environment, as there: JANIS_MAXTOK
(`cmd/llmsmoke/main.go:61-66`), JANIS_REPEAT_PENALTY and JANIS_REPEAT_LAST_N
(`engine.go:30-33`; here the penalty is off unless the variable is set).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

USAGE = """usage: janis generate --model DIR (--ids 1,2,3 | --ids-file FILE) [--temp 0] [--top-p 1] [--max-tokens 512]
                      [--seed 0] [--stop 1,107] [--dtype bfloat16|float32] [--max-cache-tokens N]
       janis generate --random CONFIG.json [--weights-seed 0] ...   (random weights instead of a folder)
       janis replay   --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   < steps.jsonl
       janis random   --config CONFIG.json --out DIR [--seed 0]     (write a folder of random weights)
       janis bench    [--steps K] [--warmup W] [--batch 8] [--context 8192] [--layers N]
       janis version"""


def _ids(text: str) -> list[int]:
    return [int(t) for t in text.replace("\n", ",").replace(" ", ",").split(",") if t.strip()]


def _env_float(name: str, default: float) -> float:
    try:
        return float(os.environ[name])
    except (KeyError, ValueError):
        return default


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ[name])
    except (KeyError, ValueError):
        return default


def cmd_generate(argv) -> int:
    ap = argparse.ArgumentParser(prog="janis generate")
    ap.add_argument("--model")
    ap.add_argument("--random", metavar="CONFIG.json")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--ids", action="append", default=[], help="a prompt as comma-separated token ids (repeatable)")
    ap.add_argument("--ids-file", help="one prompt per line, comma- or space-separated ids")
    ap.add_argument("--temp", "--temperature", dest="temp", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--max-tokens", "--max-new-tokens", dest="max_tokens", type=int,
                    default=_env_int("JANIS_MAXTOK", 512))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--stop", default=None, help="stop token ids (default: the model's end-of-sequence ids)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--max-cache-tokens", type=int, default=0)
    a = ap.parse_args(argv)
    prompts = [_ids(s) for s in a.ids]
    if a.ids_file:
        with open(a.ids_file) as f:
            prompts += [_ids(line) for line in f if line.strip()]
    if not prompts or (not a.model) == (not a.random):
        print(USAGE, file=sys.stderr)
        return 2
    import janis_b200
    need = sum((len(p) + a.max_tokens + 63) // 64 * 64 for p in prompts)
    cache_tokens = a.max_cache_tokens or min(need, 1 << 20)
    if a.model:
        eng = janis_b200.open(a.model, dtype=a.dtype, max_tokens=cache_tokens)
    else:
        with open(a.random) as f:
            eng = janis_b200.from_config(json.load(f), seed=a.weights_seed, dtype=a.dtype, max_tokens=cache_tokens)
    t0 = time.time()
    replies = eng.generate(prompts, temp=a.temp, top_p=a.top_p, max_tokens=a.max_tokens, seed=a.seed,
                           stop=_ids(a.stop) if a.stop is not None else None,
                           repeat_penalty=_env_float("JANIS_REPEAT_PENALTY", 1.0),
                           repeat_last_n=_env_int("JANIS_REPEAT_LAST_N", 64), return_replies=True)
    dt = time.time() - t0
    for r in replies:
        print(",".join(str(t) for t in r.tokens))
    n = sum(len(r.tokens) for r in replies)
    print(f"[{n} tok in {dt:.1f}s -> {n / max(dt, 1e-9):.2f} tok/s; "
          f"finish: {','.join(r.finish_reason for r in replies)}]", file=sys.stderr)
    eng.close()
    return 0


def cmd_random(argv) -> int:
    ap = argparse.ArgumentParser(prog="janis random")
    ap.add_argument("--config", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    import janis_b200
    with open(a.config) as f:
        janis_b200.write_random_model(a.out, json.load(f), seed=a.seed)
    print(a.out)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(USAGE, file=sys.stderr)
        return 2
    verb, rest = argv[0], argv[1:]
    if verb == "generate":
        return cmd_generate(rest)
    if verb == "replay":
        from .replay import main as replay_main
        return replay_main(rest)
    if verb == "random":
        return cmd_random(rest)
    if verb == "bench":
        from .benchmark import main as bench_main
        return bench_main(rest)
    if verb in ("version", "--version", "-v"):
        from . import __version__
        print("janis " + __version__)
        return 0
    print(USAGE, file=sys.stderr)
    return 2
