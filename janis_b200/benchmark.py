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
# an earlier measurement on this kind of GPU: copy bandwidth, the library's bfloat16 product as a burst and sustained
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_config(name_or_path: str) -> dict:
    path = name_or_path if os.path.exists(name_or_path) else os.path.join(_HERE, "configs", name_or_path + ".json")
    with open(path) as f:
        return json.load(f)


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        out = {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
               "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or p["bf16_tflops"])}
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
    """Bytes of cache that a decode step over sequences of these lengths reads: keys and values of every position
    a line keeps (a window of them for a windowed line), and every fixed-size state, whatever mixer asked for it."""
    from .cache.cache import KVNeed, StateNeed
    total = 0
    for needs in model.cache_line_needs():
        for need in (needs or {}).values():
            if isinstance(need, KVNeed):
                per_token = 2 * need.n_kv_heads * need.head_dim * itemsize
                total += sum(per_token * (min(n, need.window) if need.window else n) for n in lengths)
            elif isinstance(need, StateNeed):
                n = 1
                for d in need.shape:
                    n *= int(d)
                total += len(lengths) * n * torch.empty((), dtype=need.dtype).element_size()
    return total


def prefill_flops(model, n_tokens: int) -> float:
    """2 M N K of every product of a prompt step of n_tokens that asks for the last logits, plus what each
    layer's mixer says it computes beyond its products (attention: scores and weighted sums)."""
    flops = 0.0
    for name, spec in model.tensor_specs().items():
        if len(spec.shape) == 2 and "embed_tokens" not in name:
            flops += 2.0 * n_tokens * spec.shape[0] * spec.shape[1]
    for call in model.schedule:
        flops += float(model.blocks[call.layer].mixer.prompt_flops(n_tokens))
    flops += 2.0 * model.hidden * model.vocab          # the head, last position only
    return flops


# ---------------------------------------------------------------------------
# measurements
# ---------------------------------------------------------------------------

def _tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def uniform_lengths(n: int, lo: int, hi: int, seed: int) -> list[int]:
    """n seeded lengths, uniform in [lo, hi]."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def fill(engine, lengths, seed: int = 0) -> list[int]:
    """New sequences of these lengths, of seeded random tokens, by real prompt steps."""
    from .engine.step import StepEntry
    slots = [engine.alloc_slot() for _ in lengths]
    cur, cur_tok = [], 0
    batches = []
    for i, n in enumerate(lengths):
        if cur and cur_tok + n > engine.stepper.max_step_tokens:
            batches.append(cur)
            cur, cur_tok = [], 0
        cur.append(i)
        cur_tok += n
    batches.append(cur)
    for part in batches:
        engine.stepper.step([StepEntry(slots[i], _tokens(engine.model.vocab, lengths[i], seed + i), ()) for i in part])
    return slots


def measure_decode(engine, start_lengths, steps: int, warmup: int, sample_clocks: bool = False,
                   profile: bool = False, runs: int = 1) -> dict:
    """Decode tokens a second over sequences that hold `start_lengths` tokens before the first warm-up step
    (brought there by real prompt steps).  `runs` timed runs of exactly `steps` steps each, every one from the
    same lengths; the median run is reported (the reference's method: three runs, the median,
    `bench/mlx.py:41-46`).  `profile` opens the CUDA profiler range around the first two timed steps (for a
    profiler that was started with its capture off); the timing of such a run means nothing."""
    from .engine.step import StepEntry
    ops = engine.rt.ops
    batch = len(start_lengths)
    st = engine.stepper
    results = []
    clock_rows = None
    for run_no in range(max(1, runs)):
        slots = fill(engine, start_lengths)
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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks = ClockSampler() if sample_clocks else None
        if clocks:
            clocks.__enter__()
        e0.record()
        for i in range(steps):
            if profile and i == 0 and run_no == 0:
                torch.cuda.profiler.start()
            one(warmup + i)
            if profile and i == 1 and run_no == 0:
                torch.cuda.synchronize()
                torch.cuda.profiler.stop()
        e1.record()
        torch.cuda.synchronize()
        if clocks:
            clocks.__exit__()
        results.append((e0.elapsed_time(e1), clocks, int(history.cpu().sum())))
        for s in slots:
            engine.free_slot(s)
    results.sort(key=lambda r: r[0])
    ms, clocks, checksum = results[len(results) // 2]
    per_step = st.launch_counter + 1                  # kernels of one replayed step, plus argmax
    mid = [n + warmup + steps // 2 for n in start_lengths]
    bytes_step = weight_bytes(engine.model) + cache_bytes(engine.model, mid)
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "bytes_per_step": bytes_step,
            "gb_s": bytes_step / (ms / steps / 1e3) / 1e9, "gpu_launches": per_step * steps,
            "clocks": clocks.summary() if clocks else None, "tokens_checksum": checksum,
            "runs_ms_per_step": [round(r[0] / steps, 4) for r in results]}


def measure_e2e(engine, batch: int, context: int, steps: int, temp: float = 0.0, top_p: float = 1.0) -> dict:
    """The same through Engine.generate: token ids in from the host, token ids out to the host."""
    n_prompt = context - steps - 1
    prompts = [_tokens(engine.model.vocab, n_prompt, 1000 + i) for i in range(batch)]
    return measure_generate(engine, prompts, steps + 1, temp, top_p)


def measure_generate(engine, prompts, new_tokens: int, temp: float = 0.0, top_p: float = 1.0) -> dict:
    """Decode tokens a second of `Engine.generate` over these prompts, `new_tokens` each: the tokens after each
    request's first, over the time from the first token heard to the end (the reference's decode rate,
    `cmd/enginebench/main.go:172-189`), and the time to that first token."""
    t_first = [None]
    count = [0]

    def on_token(i, tok):
        if t_first[0] is None:
            torch.cuda.synchronize()
            t_first[0] = time.perf_counter()
        count[0] += 1

    # warm-up: the same call over the same lengths, so that every graph the timed call replays exists
    engine.generate(prompts, temp=temp, top_p=top_p, max_tokens=new_tokens, stop=())
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.generate(prompts, temp=temp, top_p=top_p, max_tokens=new_tokens, stop=(), on_token=on_token)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t_first[0]
    return {"tok_s": (count[0] - len(prompts)) / dt, "h2d_bytes_per_step": engine.stepper.h2d_bytes,
            "d2h_bytes_per_step": 4 * len(prompts), "first_token_ms": (t_first[0] - t0) * 1e3}


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


def fp32_check(raw: dict, bf16_engine, n_tokens: int = 256, seed: int = 0) -> dict:
    """The logits at the end of a seeded prompt from the bfloat16 engine against a true 32-bit engine over the
    same weights: the largest difference as a fraction of the largest logit."""
    import janis_b200
    from .engine.step import StepEntry
    toks = _tokens(bf16_engine.model.vocab, n_tokens, 4242)
    slot = bf16_engine.alloc_slot()
    a = bf16_engine.step([StepEntry(slot, toks, (n_tokens - 1,))]).float().cpu()
    bf16_engine.free_slot(slot)
    ref = janis_b200.from_config(raw, seed=seed, dtype="float32", max_tokens=max(64, n_tokens), max_batch=1)
    slot = ref.alloc_slot()
    b = ref.step([StepEntry(slot, toks, (n_tokens - 1,))]).float().cpu()
    ref.close()
    return {"tokens": n_tokens, "max_err": round(float((a - b).abs().max()), 5),
            "scale": round(float(b.abs().max()), 3), "same_argmax": bool(a.argmax() == b.argmax())}


def _pretty(config: str) -> str:
    name = os.path.splitext(os.path.basename(config))[0]
    return "Gemma2-" + name[len("gemma2-"):].upper() if name.startswith("gemma2-") else name


def _frac(r: dict, pk: dict) -> float:
    return round(r["gb_s"] / pk["hbm_gbs"], 4)


def run(steps: int = 256, warmup: int = 8, batch: int = 8, context: int = 8192, config: str = "gemma2-2b",
        layers: int | None = None, points=(1, 64), prefill_tokens: int = 2048, e2e: bool = True,
        profile: str = "", runs: int = 3, workloads: bool = True, prompt_lengths=None) -> dict:
    """The whole benchmark; returns the record that bench.py prints as one JSON line.

    The headline is the median of `runs` runs of exactly `steps` decode steps at `batch` sequences whose cache
    reaches `context` tokens.  `points` adds decode at other batch sizes at the same context.  `workloads` adds
    the other measurements the configurations are quoted with: decode at batch 1, 8 and 64 from prompts of
    seeded lengths uniform in [128, 2048]; the 9B sizes generating 256 tokens each for an unequal batch of 8
    prompts of lengths uniform in [64, 4096] through `Engine.generate`; the 27B sizes' prompt step of 2,048
    tokens and decode at batch 1 and 16 from prompts of 1,024; each decode point with the fraction of the
    copy bandwidth that its own lengths give it; and the bfloat16 logits of the headline model against a true
    32-bit engine."""
    import janis_b200
    raw = load_config(config)
    full_layers = raw["num_hidden_layers"]
    if layers:
        raw = dict(raw, num_hidden_layers=int(layers))
    pk, pk_kind = peaks()
    max_batch = max([batch, *points, *((64,) if workloads else ())])
    room = max(context, prefill_tokens)                 # the prefill measurement needs its own length to fit
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=max_batch * room, max_batch=max_batch,
                                 max_context=room)
    start = context - steps - warmup
    if start < 1:
        raise ValueError("context too short for the steps asked")
    # (prompt_lengths = (lo, hi): the headline run decodes from prompts of seeded lengths uniform in [lo, hi] instead)
    starts = uniform_lengths(batch, prompt_lengths[0], prompt_lengths[1], 7 + batch) if prompt_lengths else [start] * batch
    main = measure_decode(eng, starts, steps, warmup, sample_clocks=True, profile=profile == "decode",
                          runs=1 if profile else runs)
    pre = measure_prefill(eng, prefill_tokens, profile=profile == "prefill")
    pts = {}
    for b in points:
        k = max(16, steps // 2)
        r = measure_decode(eng, [context - k - warmup] * b, k, warmup)
        pts[f"decode_b{b}"] = round(r["tok_s"], 1)
        pts[f"decode_b{b}_frac"] = _frac(r, pk)
    if workloads and not profile:
        for b in (1, 8, 64):                            # prompts of seeded lengths uniform in [128, 2048]
            r = measure_decode(eng, uniform_lengths(b, 128, 2048, 7 + b), 128, warmup, runs=3)
            pts[f"decode_b{b}_u2048"] = round(r["tok_s"], 1)
            pts[f"decode_b{b}_u2048_frac"] = _frac(r, pk)
    end = measure_e2e(eng, batch, context, steps) if e2e and not profile else None
    if end and workloads:                                # and with sampling instead of the highest logit
        pts["e2e_b%d_temp0.8_top_p0.95" % batch] = round(measure_e2e(eng, batch, context, steps, 0.8, 0.95)["tok_s"], 1)
    check = fp32_check(raw, eng) if workloads and not profile else None
    cfg = eng.config
    eng.close()
    del eng
    if workloads and not profile:
        pts.update(other_sizes(pk, warmup))
    rec = {
        "metric": "decode tok/s at batch %d (%s sizes, %s)" % (
            batch, _pretty(config), "prompts of %d to %d tokens" % tuple(prompt_lengths) if prompt_lengths else "context %d" % context),
        "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": config, "layers": cfg.num_hidden_layers, "layers_of_model": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "window": cfg.sliding_window, "global_batch": batch, "seq_len": context,
                   "context_len": context, "prefill_tokens": prefill_tokens, "weights": "random seed 0",
                   "parallelism": "single", "l2": "each step reads weights+cache >> L2",
                   "timed_runs": "median of %d" % (1 if profile else runs)},
        "clocks": main["clocks"], "gpu_launches": main["gpu_launches"], "runs_ms_per_step": main["runs_ms_per_step"],
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": prefill_tokens, "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_of_sustained": round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(main["gb_s"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": _frac(main, pk), "peaks": pk_kind},
        "points": pts,
    }
    if end:
        rec["e2e"] = {"value": round(end["tok_s"], 1), "unit": "tok/s", "h2d_bytes_per_step": end["h2d_bytes_per_step"],
                      "d2h_bytes_per_step": end["d2h_bytes_per_step"]}
    if check:
        rec["fp32_check"] = check
    return rec


def other_sizes(pk: dict, warmup: int = 8) -> dict:
    """The measurements quoted for the larger configurations (all of their layers, random weights):
    9B: an unequal batch of 8 prompts of seeded lengths uniform in [64, 4096], 256 tokens generated for each,
    through `Engine.generate` (host tokens in and out); 27B: the prompt step of 2,048 tokens, and decode at batch 1
    and 16 from prompts of 1,024 tokens."""
    import janis_b200
    out = {}
    raw = load_config("gemma2-9b")
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=8 * (4096 + 256 + 64), max_batch=8,
                                 max_context=8192)
    lens = uniform_lengths(8, 64, 4096, 5)
    prompts = [_tokens(eng.model.vocab, n, 3000 + i) for i, n in enumerate(lens)]
    g = measure_generate(eng, prompts, 256)
    out["gen_9b_b8_u4096_tok_s"] = round(g["tok_s"], 1)
    out["gen_9b_b8_u4096_first_token_ms"] = round(g["first_token_ms"], 1)
    mid = [n + 128 for n in lens]
    bytes_step = weight_bytes(eng.model) + cache_bytes(eng.model, mid)
    out["gen_9b_b8_u4096_frac"] = round(bytes_step * (g["tok_s"] / 8) / 1e9 / pk["hbm_gbs"], 4)
    eng.close()
    del eng
    raw = load_config("gemma2-27b")
    eng = janis_b200.from_config(raw, seed=0, dtype="bfloat16", max_tokens=16 * 2048, max_batch=16, max_context=8192)
    pre = measure_prefill(eng, 2048, repeats=3, warmup=2)
    out["prefill_27b_tok_s"] = round(pre["tok_s"], 1)
    out["prefill_27b_frac"] = round(pre["flops"] / (pre["ms"] / 1e3) / (pk["bf16_tflops"] * 1e12), 4)
    for b in (1, 16):
        r = measure_decode(eng, [1024] * b, 64, warmup, runs=3)
        out[f"decode_27b_b{b}_p1024"] = round(r["tok_s"], 1)
        out[f"decode_27b_b{b}_p1024_frac"] = _frac(r, pk)
    eng.close()
    return out


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
    ap.add_argument("--no-workloads", action="store_true",
                    help="leave out the unequal-length decode points, the 9B and 27B measurements and the 32-bit check")
    ap.add_argument("--runs", type=int, default=3, help="timed runs of the headline; the median is reported")
    ap.add_argument("--prompt-lengths", default="", help="LO,HI: decode from prompts of seeded lengths uniform in [LO, HI] "
                    "instead of sequences that all reach --context")
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
              points=() if (a.no_points or a.profile) else points, prefill_tokens=a.prefill, profile=a.profile,
              runs=max(1, a.runs), workloads=not (a.no_workloads or a.no_points) and config == "gemma2-2b" and not a.layers,
              prompt_lengths=tuple(int(v) for v in a.prompt_lengths.split(",")) if a.prompt_lengths else None)
    print(json.dumps(rec))
    return 0
