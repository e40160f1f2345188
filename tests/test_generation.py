"""Generation and replay through their entry points: `Engine.generate`, `bin/janis generate`,
`bin/trace_run`.  GPU cases use the CUDA kernels; the `refs` cases run the same engine over the
plain kernel statements on the CPU and so test the loop, the batching and the cache together."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests.conftest import ROOT, TINY, plain_logits, random_tokens
from tests.helpers import assert_logits, make_engine, model_tol
from tests.plain import gemma2_plain as P

GPU = pytest.mark.gpu
CASES = [pytest.param("cuda", "float32", marks=GPU), pytest.param("cuda", "bfloat16", marks=GPU),
         pytest.param("refs", "float32")]


def check_greedy(plain_models, key, dtype, prompt, reply, stop=()):
    """Every token of a greedy reply is the plain model's choice for the text so far; in bfloat16 it
    may be a near-tie instead: within the model tolerance of the plain maximum."""
    cfg, w = plain_models[key]
    seq = list(prompt)
    for tok in reply:
        logits = plain_logits(plain_models, key, seq)[-1]
        assert tok not in stop
        if dtype == "float32":
            assert tok == P.sample_token(logits, 0.0, 1.0, 0.0), f"{key}: token {len(seq) - len(prompt)} of the reply"
        else:
            assert logits[tok] >= logits.max() - 2 * model_tol(dtype) * logits.abs().max()
        seq.append(tok)
    return plain_logits(plain_models, key, seq)[-1]


@pytest.mark.parametrize("on,dtype", CASES)
def test_greedy_generation_of_unequal_prompts_in_several_batches(on, dtype, model_dirs, plain_models):
    for key in (["A", "B", "B_hot"] if on == "cuda" else ["B"]):
        V = TINY[key[0]]["vocab_size"]
        eng = make_engine(model_dirs[key], dtype, on, max_tokens=6 * 64, max_batch=3)
        prompts = [random_tokens(V, n, 80 + n) for n in (5, 11, 17, 1, 70, 9, 23)]
        replies = eng.generate(prompts, temp=0.0, max_tokens=8, stop=(), return_replies=True)
        assert [r.finish_reason for r in replies] == ["length"] * len(prompts)
        for p, r in zip(prompts, replies):
            assert len(r.tokens) == 8
            check_greedy(plain_models, key, dtype, p, r.tokens)
        assert eng.cache.live_slots() == []
        eng.cache.audit()
        eng.close()


@pytest.mark.parametrize("on,dtype", CASES)
def test_stop_tokens_end_replies_early(on, dtype, model_dirs, plain_models):
    key = "B"
    V = TINY["B"]["vocab_size"]
    eng = make_engine(model_dirs[key], dtype, on, max_tokens=1024)
    prompts = [random_tokens(V, n, 90 + n) for n in (4, 12, 30)]
    free = eng.generate(prompts, temp=0.0, max_tokens=10, stop=())
    stop = {free[0][3], free[1][6]}                                   # tokens that do occur in replies
    replies = eng.generate(prompts, temp=0.0, max_tokens=10, stop=stop, return_replies=True)
    for p, f, r in zip(prompts, free, replies):
        cut = next((i for i, t in enumerate(f) if t in stop), None)
        if cut is None:
            assert r.tokens == f and r.finish_reason == "length"
        else:
            assert r.tokens == f[:cut] and r.finish_reason == "stop"
    # the configuration's own end-of-sequence ids are the default stop set
    assert set(eng.stop_tokens) == {1, 7}
    eng.close()


@pytest.mark.parametrize("on,dtype", CASES)
def test_sampled_replies_depend_on_seed_and_request_not_on_the_batch(on, dtype, model_dirs):
    key = "B_hot"
    V = TINY["B"]["vocab_size"]
    eng = make_engine(model_dirs[key], dtype, on, max_tokens=2048)
    prompts = [random_tokens(V, n, 100 + n) for n in (6, 13, 21, 9)]
    a = eng.generate(prompts, temp=0.9, top_p=0.95, seed=7, max_tokens=12, stop=())
    b = eng.generate(prompts, temp=0.9, top_p=0.95, seed=7, max_tokens=12, stop=())
    c = eng.generate(prompts, temp=0.9, top_p=0.95, seed=8, max_tokens=12, stop=())
    assert a == b and a != c
    greedy = eng.generate(prompts, temp=0.0, max_tokens=12, stop=())
    assert a != greedy
    if dtype == "float32":
        # request 0 alone draws the same numbers: its reply is the same whatever else is in the batch
        assert eng.generate(prompts[:1], temp=0.9, top_p=0.95, seed=7, max_tokens=12, stop=())[0] == a[0]
    pen = eng.generate(prompts, temp=0.0, max_tokens=12, stop=(), repeat_penalty=1.5, repeat_last_n=8)
    assert pen != greedy                                              # hot tied weights repeat themselves unless penalised
    eng.close()


def _trace(requests, prompt_lens, batch_of):
    """Step records for `requests` run in batches of `batch_of`, prompts first, then one token a step."""
    steps, n_step = [], 0
    live_peak = 0
    for b0 in range(0, len(requests), batch_of):
        ids = list(range(b0, min(len(requests), b0 + batch_of)))
        pos = {i: prompt_lens[i] for i in ids}
        entries = [{"id": f"r{i}", "tokens": requests[i][:pos[i]], "want": list(range(pos[i]))} for i in ids]
        while entries:
            done = [i for i in ids if pos[i] >= len(requests[i])]
            live_peak = max(live_peak, sum((pos[i] + 63) // 64 * 64 for i in ids))
            steps.append({"step": n_step, "entries": entries, "end": [f"r{i}" for i in done]})
            n_step += 1
            ids = [i for i in ids if i not in done]
            entries = [{"id": f"r{i}", "tokens": [requests[i][pos[i]]], "want": [0]} for i in ids]
            for i in ids:
                pos[i] += 1
    return steps, live_peak


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_user_runs_it(dtype, model_dirs, plain_models, tmp_path):
    key = "B_hot"
    V = TINY["B"]["vocab_size"]
    lens = [40, 9, 75, 1, 23, 130]
    reqs = [random_tokens(V, n, 110 + n) for n in lens]
    prompts = [max(1, n - 32) for n in lens]
    steps, peak = _trace(reqs, prompts, batch_of=3)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dirs[key], "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(peak)],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    got = {f"r{i}": [] for i in range(len(reqs))}
    for s in steps:
        arr = np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, V)
        o = 0
        for e in s["entries"]:
            got[e["id"]].append(torch.from_numpy(arr[o:o + len(e["want"])].copy()))
            o += len(e["want"])
        assert o == arr.shape[0]
    for i, r in enumerate(reqs):
        assert_logits(torch.cat(got[f"r{i}"]), plain_logits(plain_models, key, r), dtype, f"trace request {i}")


def test_replay_of_a_trace_over_the_cpu_statements_and_its_refusals(model_dirs, plain_models, tmp_path):
    """`run_trace` itself, in this process, over the engine on the plain kernel statements: the records it reads,
    the slots it takes and gives back, the files and the lines it writes, and what it refuses."""
    import io
    from janis_b200.replay import TraceError, run_trace
    key = "B"
    V = TINY["B"]["vocab_size"]
    lens = [12, 5, 37, 1, 9]
    reqs = [random_tokens(V, n, 140 + n) for n in lens]
    steps, _ = _trace(reqs, [max(1, n - 4) for n in lens], batch_of=2)
    eng = make_engine(model_dirs[key], "float32", "refs", max_tokens=4 * 64, max_batch=2)
    out, said = tmp_path / "out", io.StringIO()
    lines = [json.dumps(s) for s in steps]
    lines.insert(1, "   ")                                             # an empty line is no step
    assert run_trace(eng, lines, str(out), said) == len(steps)
    assert said.getvalue().split() == [w for s in steps for w in ("done", str(s["step"]))]
    got = {f"r{i}": [] for i in range(len(reqs))}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        path = out / f"{s['step']}.f32"
        assert path.exists() == (wanted > 0)
        if not wanted:
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(-1, V)
        assert arr.shape[0] == wanted
        o = 0
        for e in s["entries"]:
            got[e["id"]].append(torch.from_numpy(arr[o:o + len(e["want"])].copy()))
            o += len(e["want"])
    for i, r in enumerate(reqs):
        assert_logits(torch.cat(got[f"r{i}"]), plain_logits(plain_models, key, r), "float32", f"trace request {i}")
    assert eng.cache.live_slots() == [] and not list(out.glob(".*tmp"))
    # a step that wants nothing writes no file; a request that ends without having started, and a line that is
    # no record, are refused with the line's number
    quiet = [json.dumps({"step": 999, "entries": [{"id": "q", "tokens": [1, 2, 3], "want": []}], "end": ["q"]})]
    assert run_trace(eng, quiet, str(out), io.StringIO()) == 1 and not (out / "999.f32").exists()
    with pytest.raises(TraceError, match="line 1.*'zz'.*never started"):
        run_trace(eng, [json.dumps({"step": 0, "entries": [], "end": ["zz"]})], str(out), io.StringIO())
    with pytest.raises(TraceError, match="line 2: not a step record"):
        run_trace(eng, [quiet[0], "{\"step\": 1"], str(out), io.StringIO())
    assert eng.cache.live_slots() == []
    eng.cache.audit()
    eng.close()


@GPU
def test_janis_generate_command(model_dirs, plain_models):
    key = "B"
    prompt = random_tokens(TINY["B"]["vocab_size"], 9, 120)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janis"), "generate", "--model", model_dirs[key],
                        "--ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--dtype", "float32", "--stop", ""],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    reply = [int(t) for t in p.stdout.strip().split(",")]
    assert len(reply) == 5
    check_greedy(plain_models, key, "float32", prompt, reply)
    bad = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "janis"), "frobnicate"], capture_output=True, text=True)
    assert bad.returncode == 2 and "usage: janis" in bad.stderr


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_engine_from_a_configuration_alone(dtype, tmp_path):
    """Weights drawn on the device from (seed, tensor name) are the ones the random-weights folder of the same
    seed holds (drawn on the CPU): the engine's greedy reply is the plain model's over that folder."""
    import janis_b200
    janis_b200.write_random_model(str(tmp_path), TINY["B"], seed=3)
    plain = {"rnd": P.load_folder(str(tmp_path))}
    eng = janis_b200.from_config(TINY["B"], seed=3, dtype=dtype, max_tokens=256)
    prompt = random_tokens(TINY["B"]["vocab_size"], 21, 130)
    out = eng.generate([prompt], max_tokens=4, stop=())
    assert len(out[0]) == 4
    check_greedy(plain, "rnd", dtype, prompt, out[0])
    eng.close()
    with pytest.raises(RuntimeError, match="closed"):
        eng.generate([[1]])


@GPU
def test_a_given_up_wait_is_reported_by_the_engine(tmp_path):
    """A CTA that gives up a bounded wait returns without its result.  The engine reads the libraries' counters
    wherever it waits for tokens anyway: a count that has grown ends `generate` with an error instead of
    tokens nobody should trust; afterwards the engine works as before.  (Head size 96: a library whose
    counter no other test expects to be zero; the probe is a one-warp kernel whose barrier nothing completes.)"""
    import janis_b200
    from janis_b200.kernels import ops
    cfg = dict(TINY["B"], head_dim=96, query_pre_attn_scalar=96)
    eng = janis_b200.from_config(cfg, seed=4, dtype="bfloat16", max_tokens=512)
    prompts = [random_tokens(cfg["vocab_size"], n, 140 + n) for n in (9, 30)]
    first = eng.generate(prompts, max_tokens=5, stop=())
    assert ops.attn_wait_probe(96, tries=32) == 1
    with pytest.raises(ops.KernelError, match="gave up a bounded wait"):
        eng.generate(prompts, max_tokens=5, stop=())
    assert eng.cache.live_slots() == []
    eng.cache.audit()
    assert eng.generate(prompts, max_tokens=5, stop=()) == first
    assert ops.attn_wait_probe(96, tries=32) == 1
    with pytest.raises(ops.KernelError, match="gave up a bounded wait"):
        eng.check_health()
    eng.check_health()
    eng.close()
