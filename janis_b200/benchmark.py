"""Measuring decode and prompt throughput of a model with random weights on one GPU.

The numbers the reference's benchmark reports per turn are context tokens, the time
to the first token and decode tokens a second = (tokens - 1) / (t_last - t_first)
(`cmd/enginebench/main.go:172-189`, `:315-336`; `bench/mlx.py:20-41`).  The same
two quantities are measured here on seeded synthetic tokens:

* decode: `batch` sequences are brought to the wanted context length by real prompt
  steps, then `warmup + steps` decode steps run; tokens stay on the device (the next
  token is picked there and fed to the next step) and the timed steps are bracketed by
  CUDA events.  Every step reads all weights and the cache of the live sequences, far
  more than the L2 holds, so nothing needs flushing between steps.
* end to end: the same through `Engine.generate`: per step the host sends the step's
  tables from pinned memory and reads the chosen tokens back.
* prompt: one step over a prompt of 2,048 tokens that returns the last logits.

Each comes with the fraction of its roofline: bytes that a decode step must read
(every weight once, and the cache of the live requests) over time against the HBM
copy bandwidth; the prompt step's floating-point operations over time against the
bfloat16 matrix peak.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_HERE)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}      # an earlier measurement on this kind of GPU


def load_config(name_or_path: str) -> dict:
    path = name_or_path if os.path.exists(name_or_path) else os.path.join(_HERE, "configs", name_or_path + ".json")
    with open(path) as f:
        return json.load(f)


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {"hbm_gbs": float(p["hbm_gbs"]),
               "bf16_tflops": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"])}
        return out, "measured"
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in a loop while a region is timed: SM clock and the reasons for slowing down."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.rows: list[list[str]] = []
        self.proc = None
        self.device_index = device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": int(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ---------------------------------------------------------------------------
# what a step must read and compute
# ---------------------------------------------------------------------------

def weight_bytes(model, itemsize: int = 2) -> int:
    """Bytes of every tensor a decode step reads once (the tied table counts once: the head reads all of
    it, the embedding a row per sequence)."""
    total = 0
    for spec in model.tensor_specs().values():
        n = 1
        for s in spec.shape:
            n *= s
        total += n * (4 if len(spec.shape) == 1 else itemsize)
    return total


def cache_bytes(model, lengths, itemsize: int = 2) -> int:
    """Bytes of keys and values that a decode step over sequences of these lengths reads."""
    total = 0
    for needs in model.cache_line_needs():
        kv = needs.get("kv")
        if kv is None:
            continue
        per_token = 2 * kv.n_kv_heads * kv.head_dim * itemsize
        for n in lengths:
            total += per_token * (min(n, kv.window) if kv.window else n)
    return total


def prefill_flops(model, n_tokens: int) -> float:
    """2 M N K of every product of a prompt step of n_tokens that asks for the last logits, plus the
    two products of attention over the visible keys."""
    flops = 0.0
    for name, spec in model.tensor_specs().items():
        if len(spec.shape) == 2 and "embed_tokens" not in name:
            flops += 2.0 * n_tokens * spec.shape[0] * spec.shape[1]
    for blk in (model.blocks[c.layer] for c in model.schedule):
        m = blk.mixer
        w = m.window or n_tokens
        visible = sum(min(i + 1, w) for i in range(n_tokens))
        flops += 4.0 * m.n_heads * m.head_dim * visible
    flops += 2.0 * model.hidden * model.vocab          # the head, last position only
    return flops


# ---------------------------------------------------------------------------
# measurements
# ---------------------------------------------------------------------------

def _tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def fill(engine, batch: int, length: int, seed: int = 0) -> list[int]:
    """`batch` new sequences of `length` seeded random tokens each, by real prompt steps."""
    from .engine.step import StepEntry
    slots = [engine.alloc_slot() for _ in range(batch)]
    per_step = max(1, engine.stepper.max_step_tokens // max(length, 1))
    for i in range(0, batch, per_step):
        part = slots[i:i + per_step]
        engine.stepper.step([StepEntry(s, _tokens(engine.model.vocab, length, seed + i + j), ())
                             for j, s in enumerate(part)])
    return slots


def measure_decode(engine, batch: int, context: int, steps: int, warmup: int, sample_clocks: bool = False,
                   profile: bool = False) -> dict:
    """Decode tokens a second at `batch` sequences whose cache grows to `context` tokens by the last step.
    `profile` opens the CUDA profiler range around the first two timed steps (for a profiler that was
    started with its capture off); the timing of such a run means nothing."""
    from .engine.step import StepEntry
    ops = engine.rt.ops
    start_len = context - steps - warmup
    if start_len < 1:
        raise ValueError("context too short for the steps asked")
    slots = fill(engine, batch, start_len)
    st = engine.stepper
    toks = st.token_buffer(batch)
    toks.copy_(torch.tensor(_tokens(engine.model.vocab, batch, 99), dtype=torch.int32))
    entries = [StepEntry(s, (0,), (0,)) for s in slots]
    history = torch.zeros((steps + warmup, batch), dtype=torch.int32, device=engine.rt.device)

    def one(i):
        logits = st.step(entries, copy=False, tokens_on_device=True)
        ops.argmax(logits, toks)                      # the next step's tokens, picked on the device
        history[i].copy_(toks)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = ops.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    clocks = ClockSampler() if sample_clocks else None
    if clocks:
        clocks.__enter__()
    e0.record()
    for i in range(steps):
        if profile and i == 0:
            torch.cuda.profiler.start()
        one(warmup + i)
        if profile and i == 1:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
    e1.record()
    torch.cuda.synchronize()
    if clocks:
        clocks.__exit__()
    ms = e0.elapsed_time(e1)
    per_step = st.launch_counter + 1                  # kernels of one replayed step, plus argmax
    mid = start_len + warmup + steps // 2
    bytes_step = weight_bytes(engine.model) + cache_bytes(engine.model, [mid] * batch)
    tokens_out = history.cpu()
    for s in slots:
        engine.free_slot(s)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "bytes_per_step": bytes_step,
            "gb_s": bytes_step / (ms / steps / 1e3) / 1e9, "gpu_launches": per_step * steps,
            "clocks": clocks.summary() if clocks else None, "tokens_checksum": int(tokens_out.sum()),
            "eager_launches": ops.launch_count() - launches0}


def measure_e2e(engine, batch: int, context: int, steps: int) -> dict:
    """The same through Engine.generate: token ids in from the host, token ids out to the host."""
    n_prompt = context - steps - 1
    prompts = [_tokens(engine.model.vocab, n_prompt, 1000 + i) for i in range(batch)]
    t_first = [None]
    count = [0]

    def on_token(i, tok):
        if t_first[0] is None:
            torch.cuda.synchronize()
            t_first[0] = time.perf_counter()
        count[0] += 1

    # warm-up: the same call over the same lengths, so that every graph the timed call replays exists
    engine.generate(prompts, temp=0.0, max_tokens=steps + 1, stop=())
    torch.cuda.synchronize()
    engine.generate(prompts, temp=0.0, max_tokens=steps + 1, stop=(), on_token=on_token)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_first[0]
    return {"tok_s": (count[0] - batch) / dt, "h2d_bytes_per_step": engine.stepper.h2d_bytes,
            "d2h_bytes_per_step": 4 * batch}


def measure_prefill(engine, n_tokens: int, repeats: int = 5, warmup: int = 3, profile: bool = False) -> dict:
    from .engine.step import StepEntry
    times = []
    for r in range(warmup + repeats):
        slot = engine.alloc_slot()
        toks = _tokens(engine.model.vocab, n_tokens, 500 + r)
        torch.cuda.synchronize()
        last = profile and r == warmup + repeats - 1
        if last:
            torch.cuda.profiler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.stepper.step([StepEntry(slot, toks, (n_tokens - 1,))])
        e1.record()
        torch.cuda.synchronize()
        if last:
            torch.cuda.profiler.stop()
        if r >= warmup:
            times.append(e0.elapsed_time(e1))
        engine.free_slot(slot)
    ms = float(np.median(times))
    return {"tok_s": n_tokens / (ms / 1e3), "ms": ms, "flops": prefill_flops(engine.model, n_tokens)}


def _pretty(config: str) -> str:
    name = os.path.splitext(os.path.basename(config))[0]
    return "Gemma2-" + name[len("gemma2-"):].upper() if name.startswith("gemma2-") else name


def run(steps: int = 256, warmup: int = 8, batch: int = 8, context: int = 8192, config: str = "gemma2-2b",
        layers: int | None = None, points=(1, 64), prefill_tokens: int = 2048, e2e: bool = True,
        profile: str = "") -> dict:
    """The whole benchmark; returns the record that bench.py prints as one JSON line."""
    import janis_b200
    raw = load_config(config)
    full_layers = raw["num_hidden_layers"]
    if layers:
        raw = dict(raw, num_hidden_layers=int(layers))
    pk, pk_kind = peaks()
    max_batch = max([batch, *points])
    room = max(context, prefill_tokens)                 # the prefill measurement needs its own length to fit
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=max_batch * room, max_batch=max_batch,
                                 max_context=room)
    main = measure_decode(eng, batch, context, steps, warmup, sample_clocks=True, profile=profile == "decode")
    pre = measure_prefill(eng, prefill_tokens, profile=profile == "prefill")
    pts = {}
    for b in points:
        pts[f"decode_b{b}"] = round(measure_decode(eng, b, context, max(16, steps // 2), warmup)["tok_s"], 1)
    end = measure_e2e(eng, batch, context, steps) if e2e and not profile else None
    cfg = eng.config
    rec = {
        "metric": "decode tok/s at batch %d (%s sizes, context %d)" % (batch, _pretty(config), context),
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": config, "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "window": cfg.sliding_window, "global_batch": batch, "seq_len": context,
                   "context_len": context, "prefill_tokens": prefill_tokens, "weights": "random seed 0",
                   "parallelism": "single", "l2": "each step reads weights+cache >> L2"},
        "clocks": main["clocks"], "gpu_launches": main["gpu_launches"],
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": prefill_tokens, "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(main["gb_s"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main["gb_s"] / pk["hbm_gbs"], 4), "peaks": pk_kind},
        "points": pts,
    }
    if end:
        rec["e2e"] = {"value": round(end["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": end["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": end["d2h_bytes_per_step"]}
    eng.close()
    return rec


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="janis bench")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256,
                    help="timed decode steps (0.6 s at the default sizes: several clock samples, and the first and last step of the end-to-end run weigh little)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="janis_b200")
    ap.add_argument("--batch", default="8", help="sequences decoded together; a list (8,1,64) also times the others")
    ap.add_argument("--context", "--ctx", dest="context", type=int, default=8192)
    ap.add_argument("--prefill", type=int, default=2048, help="tokens of the timed prompt step")
    ap.add_argument("--json", action="store_true", help="accepted for familiarity: the record is always one JSON line")
    ap.add_argument("--config", default="gemma2-2b", help="2b, 9b, 27b, gemma2-2b ... or a config.json")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--profile", choices=["decode", "prefill"], default="",
                    help="open the CUDA profiler range around two timed decode steps, or the last prompt step")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Go module (no Go toolchain here, "
                          "nothing pip can install) and its Gemma2 loads MLX 4-bit checkpoints on Apple hardware only"}))
        return 0
    if a.gpus != 1:
        print(f"janis_b200 is a one-GPU library: --gpus {a.gpus} is not supported")
        return 2
    try:
        batches = [int(b) for b in str(a.batch).split(",") if b.strip()]
    except ValueError:
        batches = []
    if not batches or min(batches) < 1:
        print(f"--batch wants positive integers, found {a.batch!r}")
        return 2
    points = tuple(batches[1:]) if len(batches) > 1 else (1, 64)
    config = a.config if (os.path.exists(a.config) or a.config.startswith("gemma2-")) else "gemma2-" + a.config
    rec = run(a.steps, max(3, a.warmup), batches[0], a.context, config, a.layers or None,
              points=() if (a.no_points or a.profile) else points, prefill_tokens=a.prefill, profile=a.profile)
    print(json.dumps(rec))
    return 0
