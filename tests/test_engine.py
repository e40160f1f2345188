"""The engine against the plain implementation: whole prompts, the last 32 tokens one
by one, unequal batches whose shorter requests end earlier with slots used again,
long decoding, the first tokens of a sequence.

Every case runs on the GPU (`-m gpu`: the CUDA kernels, float32 and bfloat16) and,
as a check of the host side alone, on the CPU over the plain kernel statements
(`on="refs"`, float32, the smaller model).
"""
from __future__ import annotations

import pytest
import torch

from tests.conftest import TINY, plain_logits, random_tokens
from tests.helpers import assert_logits, make_engine, run_requests

GPU = pytest.mark.gpu
CASES = [pytest.param("cuda", "float32", marks=GPU), pytest.param("cuda", "bfloat16", marks=GPU),
         pytest.param("refs", "float32")]
MODELS = ["A", "B", "A_hot", "B_hot"]


def vocab_of(key):
    return TINY[key[0]]["vocab_size"]


def models_for(on):
    return MODELS if on == "cuda" else ["A_hot", "B"]


@pytest.fixture(scope="module")
def engines(model_dirs):
    """Engines are expensive to open: one per (model, dtype, backend), reused; every test leaves
    the cache empty (audited)."""
    made = {}

    def get(key, dtype, on, **kw):
        k = (key, dtype, on, tuple(sorted(kw.items())))
        if k not in made:
            made[k] = make_engine(model_dirs[key], dtype, on, **kw)
        return made[k]

    yield get
    for e in made.values():
        e.close()


@pytest.mark.parametrize("on,dtype", CASES)
def test_each_request_alone_and_whole(on, dtype, engines, plain_models):
    for key in models_for(on):
        eng = engines(key, dtype, on, max_tokens=1024)
        for n, seed in ((1, 1), (5, 2), (17, 3), (64, 4), (65, 5), (140, 6)):
            req = random_tokens(vocab_of(key), n, seed)
            got = run_requests(eng, [req], [n])[0]
            assert_logits(got, plain_logits(plain_models, key, req), dtype, f"{key} whole n={n}")
        assert eng.cache.live_slots() == []


@pytest.mark.parametrize("on,dtype", CASES)
def test_last_32_tokens_one_by_one(on, dtype, engines, plain_models):
    for key in models_for(on):
        eng = engines(key, dtype, on, max_tokens=1024)
        for n, seed in ((33, 7), (40, 8), (96, 9), (150, 10)):
            req = random_tokens(vocab_of(key), n, seed)
            got = run_requests(eng, [req], [n - 32])[0]
            assert_logits(got, plain_logits(plain_models, key, req), dtype, f"{key} last-32 n={n}")


@pytest.mark.parametrize("on,dtype", CASES)
def test_unequal_batches_one_after_another(on, dtype, engines, plain_models):
    """Batches of 3 and 4 requests of unequal lengths; the shorter ones end earlier; a cache that
    holds one batch at a time, so every slot and page is used again by a later batch."""
    lens = [5, 11, 17, 1, 9, 23, 40, 70, 3, 131, 64, 2]
    prompts = [3, 11, 9, 1, 2, 20, 40, 38, 1, 100, 63, 1]
    for key in models_for(on):
        reqs = [random_tokens(vocab_of(key), n, 20 + i) for i, n in enumerate(lens)]
        for max_live in (3, 4):
            eng = engines(key, dtype, on, max_tokens=5 * 64, max_batch=4)
            got = run_requests(eng, reqs, prompts, max_live=max_live)
            for i, (g, r) in enumerate(zip(got, reqs)):
                assert_logits(g, plain_logits(plain_models, key, r), dtype,
                              f"{key} batch of {max_live}, request {i} (len {lens[i]}, prompt {prompts[i]})")
            assert eng.cache.live_slots() == []


@pytest.mark.parametrize("on,dtype", CASES)
def test_long_decoding_from_a_short_prompt(on, dtype, engines, plain_models):
    """3 prompt tokens, then 200 single-token steps: page borders, ring wrap-around (windows of 8
    and 16 live in rings of 64), and a second request beside it that starts longer and ends sooner."""
    for key in models_for(on):
        reqs = [random_tokens(vocab_of(key), 203, 40), random_tokens(vocab_of(key), 90, 41)]
        eng = engines(key, dtype, on, max_tokens=1024)
        got = run_requests(eng, reqs, [3, 70])
        for i, (g, r) in enumerate(zip(got, reqs)):
            assert_logits(g, plain_logits(plain_models, key, r), dtype, f"{key} long decode, request {i}")


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("graphs", [True, False])
def test_a_ring_of_whole_pages_wraps(on, dtype, graphs, engines, plain_models):
    """A window of 128 = two cache pages, as the real window of 4096 is a whole number of pages: a prompt of 300
    tokens (more than two rings: only its last 128 are stored), then 160 single-token steps across two wraps of
    the ring, beside a shorter request; twice, so the second round finds the slots and pages used."""
    if on != "cuda" and not graphs:
        pytest.skip("the CPU statements have no graphs to switch off")
    key = "D_hot"
    V = vocab_of(key)
    eng = engines(key, dtype, on, max_tokens=1024, use_graphs=graphs)
    for round_ in range(2):
        reqs = [random_tokens(V, 460, 600 + round_), random_tokens(V, 140, 610 + round_)]
        got = run_requests(eng, reqs, [300, 20])
        for i, (g, r) in enumerate(zip(got, reqs)):
            assert_logits(g, plain_logits(plain_models, key, r), dtype, f"{key} ring of two pages, round {round_}, request {i}")
    assert eng.cache.live_slots() == []


@pytest.mark.parametrize("on,dtype", CASES)
def test_first_tokens_of_a_sequence(on, dtype, engines, plain_models):
    """A prompt of one token, then tokens 2..12 one by one, beside a request that starts with two."""
    for key in models_for(on):
        reqs = [random_tokens(vocab_of(key), 12, 50), random_tokens(vocab_of(key), 12, 51)]
        eng = engines(key, dtype, on, max_tokens=256)
        got = run_requests(eng, reqs, [1, 2])
        for i, (g, r) in enumerate(zip(got, reqs)):
            assert_logits(g, plain_logits(plain_models, key, r), dtype, f"{key} first tokens, request {i}")


@pytest.mark.parametrize("on,dtype", CASES)
def test_padding_and_company_change_nothing(on, dtype, engines, plain_models):
    """The same request alone, in a batch of 2, and in a batch of 9 (padded to 16 rows on the GPU):
    the same logits beyond rounding; in float32 the decode rows are bit-equal."""
    key = "B_hot" if on == "cuda" else "B"
    eng = engines(key, dtype, on, max_tokens=2048)
    req = random_tokens(vocab_of(key), 40, 60)
    others = [random_tokens(vocab_of(key), 10 + 3 * i, 61 + i) for i in range(8)]
    alone = run_requests(eng, [req], [20])[0]
    pair = run_requests(eng, [req, others[0]], [20, 5])[0]
    nine = run_requests(eng, [req] + others, [20] + [4] * 8)[0]
    ref = plain_logits(plain_models, key, req)
    for name, g in (("alone", alone), ("pair", pair), ("nine", nine)):
        assert_logits(g, ref, dtype, f"{key} {name}")
    if dtype == "float32":
        assert torch.equal(alone[20:], pair[20:]) and torch.equal(alone[20:], nine[20:])


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("n_live", [17, 33, 64])
def test_decode_batches_of_many_sequences(on, dtype, n_live, engines, plain_models):
    """Decode steps of 17, 33 and 64 live sequences of unequal lengths (more rows than the skinny products
    take: library products inside the recorded step, the activation as a kernel of its own, the tensor-core
    product for the logits, batches padded to a multiple of 8); the shorter requests end earlier, so the
    batch shrinks through every padded size on its way down."""
    for key in (["B_hot", "C"] if on == "cuda" else ["B"]):
        V = vocab_of(key)
        g = torch.Generator().manual_seed(900 + n_live)
        lens = torch.randint(4, 80, (n_live,), generator=g).tolist()
        lens[0], lens[1] = 140, 3                       # one far beyond the windows, one very short
        prompts = [max(1, n - int(torch.randint(1, 12, (1,), generator=g))) for n in lens]
        reqs = [random_tokens(V, n, 910 + i) for i, n in enumerate(lens)]
        eng = engines(key, dtype, on, max_tokens=n_live * 192, max_batch=n_live)
        got = run_requests(eng, reqs, prompts)
        for i, (gi, r) in enumerate(zip(got, reqs)):
            assert_logits(gi, plain_logits(plain_models, key, r), dtype,
                          f"{key} batch of {n_live}, request {i} (len {lens[i]}, prompt {prompts[i]})")
        assert eng.cache.live_slots() == []


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_decode_batch_beyond_the_recorded_sizes(on, dtype, engines, plain_models):
    """More sequences than a recorded decode step holds (256): such a step is launched kernel by kernel with
    tables of its own."""
    key = "A_hot" if on == "cuda" else "A_hot"
    V = vocab_of(key)
    n_live = 260
    g = torch.Generator().manual_seed(77)
    lens = torch.randint(3, 9, (n_live,), generator=g).tolist()
    lens[5] = 30
    reqs = [random_tokens(V, n, 1300 + i) for i, n in enumerate(lens)]
    eng = engines(key, dtype, on, max_tokens=n_live * 64, max_batch=n_live)
    got = run_requests(eng, reqs, [n - 2 for n in lens])
    for i, (gi, r) in enumerate(zip(got, reqs)):
        assert_logits(gi, plain_logits(plain_models, key, r), dtype, f"{key} batch of {n_live}, request {i}")
    assert eng.cache.live_slots() == []


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_prompt_step_cut_into_pieces(on, dtype, engines, plain_models):
    """A prompt step of more tokens than `max_step_tokens` runs as pieces cut at sequence borders; logits are
    wanted at places in every piece (and at none in one sequence), and come back in the order of the entries."""
    from janis_b200 import StepEntry
    key = "B_hot" if on == "cuda" else "B"
    V = vocab_of(key)
    lens = [30, 25, 40, 10, 70, 3, 50]                  # pieces of at most 50 tokens: 30 | 25 | 40 10 | 70 | 3 | 50
    want = [[0, 29], [24], list(range(40)), [], [5, 69], [0, 1, 2], [49]]
    reqs = [random_tokens(V, n + 2, 1500 + i) for i, n in enumerate(lens)]
    eng = engines(key, dtype, on, max_tokens=2048, max_step_tokens=50)
    slots = [eng.alloc_slot() for _ in reqs]
    out = eng.step([StepEntry(s, r[:n], w) for s, r, n, w in zip(slots, reqs, lens, want)])
    assert out.shape[0] == sum(len(w) for w in want)
    o = 0
    for i, (r, w) in enumerate(zip(reqs, want)):
        if w:
            assert_logits(out[o:o + len(w)], plain_logits(plain_models, key, r)[w], dtype, f"{key} cut step, request {i}")
        o += len(w)
    for t in range(2):                                  # and the cache holds every piece's keys
        out = eng.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, reqs, lens)])
        for i, (r, n) in enumerate(zip(reqs, lens)):
            assert_logits(out[i:i + 1], plain_logits(plain_models, key, r)[n + t:n + t + 1], dtype,
                          f"{key} after a cut step, request {i} token {t}")
    for s in slots:
        eng.free_slot(s)
    eng.cache.audit()


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("chunk", [7, 64, 100])
def test_a_prompt_that_comes_in_pieces(on, dtype, chunk, engines, plain_models):
    """A prompt fed in steps of `chunk` tokens onto what the steps before left in the cache (the reference's
    session feeds its prompt so, `qwen/session.go:272-303`): the logits at every position are the plain model's
    over the whole sequence.  Pieces end inside, on and beyond a cache page, straddle the windows (8, 16, 40: a
    piece is longer than a ring's window, and shorter), two requests of unequal lengths run side by side, the
    shorter ends earlier, tokens one by one follow over the same cache, and the slots are used again."""
    from janis_b200 import StepEntry
    for key in (["A_hot", "B_hot", "C"] if on == "cuda" else ["B"]):
        V = vocab_of(key)
        eng = engines(key, dtype, on, max_tokens=1024)
        for round_ in range(2):
            lens = [230 + round_, 93]
            reqs = [random_tokens(V, n + 3, 1700 + 10 * round_ + i) for i, n in enumerate(lens)]
            got = [[] for _ in reqs]
            slots = [eng.alloc_slot() for _ in reqs]
            pos = [0, 0]
            while any(p < n for p, n in zip(pos, lens)):
                live = [i for i in range(len(reqs)) if pos[i] < lens[i]]
                take = [min(chunk, lens[i] - pos[i]) for i in live]
                out = eng.step([StepEntry(slots[i], reqs[i][pos[i]:pos[i] + t], list(range(t))) for i, t in zip(live, take)])
                o = 0
                for i, t in zip(live, take):
                    got[i].append(out[o:o + t].cpu())
                    o += t
                    pos[i] += t
            for t in range(3):
                out = eng.step([StepEntry(slots[i], [reqs[i][lens[i] + t]], [0]) for i in range(len(reqs))])
                for i in range(len(reqs)):
                    got[i].append(out[i:i + 1].cpu())
            for i, r in enumerate(reqs):
                assert_logits(torch.cat(got[i]), plain_logits(plain_models, key, r), dtype,
                              f"{key} pieces of {chunk}, round {round_}, request {i}")
            for sl in slots:
                eng.free_slot(sl)
            eng.cache.audit()


@pytest.mark.parametrize("on,dtype", CASES)
def test_new_sequences_beside_ones_that_go_on(on, dtype, engines, plain_models):
    """One step that starts a sequence, continues another by several tokens and a third by one token."""
    from janis_b200 import StepEntry
    key = "B_hot" if on == "cuda" else "B"
    V = vocab_of(key)
    eng = engines(key, dtype, on, max_tokens=1024)
    reqs = [random_tokens(V, n, 1800 + i) for i, n in enumerate((90, 50, 30))]
    want = [plain_logits(plain_models, key, r) for r in reqs]
    s0, s1, s2 = (eng.alloc_slot() for _ in range(3))
    eng.step([StepEntry(s0, reqs[0][:41], []), StepEntry(s1, reqs[1][:20], [])])
    out = eng.step([StepEntry(s0, reqs[0][41:90], list(range(49))), StepEntry(s1, [reqs[1][20]], [0]),
                    StepEntry(s2, reqs[2], [0, 29])])
    assert_logits(out[:49], want[0][41:90], dtype, f"{key} mixed step, continued by 49")
    assert_logits(out[49:50], want[1][20:21], dtype, f"{key} mixed step, continued by 1")
    assert_logits(out[50:], want[2][[0, 29]], dtype, f"{key} mixed step, new")
    for sl in (s0, s1, s2):
        eng.free_slot(sl)
    eng.cache.audit()


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphs_and_plain_launches_agree(dtype, model_dirs, plain_models):
    key = "A_hot"
    reqs = [random_tokens(vocab_of(key), n, 70 + n) for n in (30, 75, 12)]
    outs = []
    for graphs in (True, False):
        eng = make_engine(model_dirs[key], dtype, "cuda", max_tokens=1024, use_graphs=graphs)
        outs.append(run_requests(eng, reqs, [10, 70, 1]))
        eng.close()
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [True, False])
def test_overlapped_and_plain_launches_agree(dtype, graphs, model_dirs):
    """Kernels whose CTAs arrive while their predecessor still runs give the bits of serial launches: a
    kernel that read its input before the wait, or wrote before its predecessor had read, would differ."""
    from janis_b200.kernels import ops
    key = "B_hot"
    reqs = [random_tokens(vocab_of(key), n, 170 + n) for n in (41, 9, 77, 130)]
    outs = []
    try:
        for overlap in (True, False):
            ops.set_overlap(overlap)
            eng = make_engine(model_dirs[key], dtype, "cuda", max_tokens=2048, use_graphs=graphs)
            for _ in range(3):                      # several rounds: slots, graphs and buffers are used again
                outs.append(run_requests(eng, reqs, [24, 1, 40, 64]))
            eng.close()
    finally:
        ops.set_overlap(True)
    half = len(outs) // 2
    for with_overlap, without in zip(outs[:half], outs[half:]):
        for a, b in zip(with_overlap, without):
            assert torch.equal(a, b)


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_several_tiles_at_head_size_64(dtype, engines, plain_models):
    """A head size that the tcgen05 prompt kernel takes: prompts of several tiles of queries (some shared between
    CTAs), alone and in an unequal batch, then tokens one by one over the same cache."""
    key = "C_hot"
    eng = engines(key, dtype, "cuda", max_tokens=2048)
    reqs = [random_tokens(vocab_of(key), n, 300 + n) for n in (330, 129, 64, 200)]
    got = run_requests(eng, reqs, [300, 129, 1, 180])
    for g, r in zip(got, reqs):
        assert_logits(g, plain_logits(plain_models, key, r), dtype, f"{key} n={len(r)}")
    alone = run_requests(eng, [reqs[0]], [330])[0]
    assert_logits(alone, plain_logits(plain_models, key, reqs[0]), dtype, f"{key} alone")
    assert eng.cache.live_slots() == []


@GPU
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A_hot", "B_hot", "C_hot"])
def test_short_prompt_steps_replayed_from_graphs(key, dtype, model_dirs, plain_models):
    """Short prompt steps whose padded shape has come before run from a CUDA graph: the first batch kernel by
    kernel, the second recorded, the others replayed.  Unequal prompts (some longer than the window), a batch
    that fills its padded shape exactly, padding tokens and padding sequences, the logits at the prompts' ends
    and at the tokens decoded after them over the same cache, slots used again; and a step that wants no logits."""
    from janis_b200 import StepEntry
    eng = make_engine(model_dirs[key], dtype, "cuda", max_tokens=2048)
    V = vocab_of(key)
    poison = lambda: eng.stepper.ws.fill(float("nan"))      # a step must write every row it reads, padding included
    batches = [(30, 75, 12), (41, 50, 33), (64, 64), (1, 100, 20), (3, 2, 1), (120,)]
    for b, lens in enumerate(batches):
        reqs = [random_tokens(V, n + 3, 400 + 10 * b + i) for i, n in enumerate(lens)]
        want = [plain_logits(plain_models, key, r) for r in reqs]
        slots = [eng.alloc_slot() for _ in reqs]
        poison()
        out = eng.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lens)])
        for i, n in enumerate(lens):
            assert_logits(out[i:i + 1], want[i][n - 1:n], dtype, f"{key} batch {b} prompt {i}")
        for t in range(3):
            poison()
            out = eng.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, reqs, lens)])
            for i, n in enumerate(lens):
                assert_logits(out[i:i + 1], want[i][n + t:n + t + 1], dtype, f"{key} batch {b} request {i} token {t}")
        for s in slots:
            eng.free_slot(s)
        eng.cache.audit()
    # the first four batches share a padded shape: one graph; the last two have one each, seen once: none
    assert len(eng.stepper._prompt_graphs) == 1
    # a prompt step that wants nothing, twice (the second is recorded), then a token over what it left
    req = random_tokens(V, 50, 477)
    want = plain_logits(plain_models, key, req)
    for _ in range(3):
        slot = eng.alloc_slot()
        assert eng.step([StepEntry(slot, req[:49], [])]) is None
        out = eng.step([StepEntry(slot, [req[49]], [0])])
        assert_logits(out, want[49:50], dtype, f"{key} after a prompt step without logits")
        eng.free_slot(slot)
    assert len(eng.stepper._prompt_graphs) == 2
    eng.close()
