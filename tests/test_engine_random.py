"""Random traffic through the step function against the plain implementation: seeded scenarios of
unequal requests, prompt cuts, batch sizes and early enders, so that slots, pages and rings are used
again in orders no hand-written case thinks of.  On the CPU over the plain kernel statements (float32)
and on the GPU in both dtypes."""
from __future__ import annotations

import random

import pytest

from tests.conftest import TINY, plain_logits, random_tokens
from tests.helpers import assert_logits, make_engine, run_requests

GPU = pytest.mark.gpu


def scenario(rng: random.Random, vocab: int, longest: int):
    n = rng.randint(1, 5)
    reqs, cuts = [], []
    for i in range(n):
        length = rng.choice([1, 2, rng.randint(3, longest), rng.randint(3, longest)])
        reqs.append(random_tokens(vocab, length, rng.randint(0, 10 ** 6)))
        cuts.append(rng.randint(1, length))            # tokens that come in the prompt step; the rest one by one
    return reqs, cuts, rng.randint(1, n)


@pytest.mark.parametrize("on,dtype,key,rounds,longest", [
    pytest.param("refs", "float32", "A_hot", 6, 40),
    pytest.param("refs", "float32", "B", 4, 50),
    pytest.param("cuda", "float32", "A_hot", 60, 90, marks=GPU),
    pytest.param("cuda", "float32", "B_hot", 25, 120, marks=GPU),
    pytest.param("cuda", "bfloat16", "A_hot", 25, 90, marks=GPU),
    pytest.param("cuda", "bfloat16", "B_hot", 60, 120, marks=GPU),
    pytest.param("cuda", "bfloat16", "C_hot", 15, 300, marks=GPU),
])
def test_random_traffic(on, dtype, key, rounds, longest, model_dirs, plain_models):
    rng = random.Random(f"{on}-{dtype}-{key}")
    vocab = TINY[key[0]]["vocab_size"]
    eng = make_engine(model_dirs[key], dtype, on, max_tokens=5 * 320 + 64)
    try:
        for round_no in range(rounds):
            reqs, cuts, live = scenario(rng, vocab, longest)
            got = run_requests(eng, reqs, cuts, max_live=live)
            for i, (g, r) in enumerate(zip(got, reqs)):
                assert_logits(g, plain_logits(plain_models, key, r), dtype,
                              f"{key} round {round_no} request {i} (len {len(r)}, cut {cuts[i]}, live {live})")
            assert eng.cache.live_slots() == []
            eng.cache.audit()
    finally:
        eng.close()
