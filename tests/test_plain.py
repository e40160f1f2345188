"""The plain implementation itself: hand values in the manner of the reference's op tests
(`cpu/cpu_test.go:18-149`, tolerance 1e-4), properties that pin the formulas down, and
float32 against float64."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from tests.conftest import plain_logits, random_tokens
from tests.plain import gemma2_plain as P


def test_softmax_hand_values():
    p = P.softmax_rows(torch.tensor([[1.0, 2.0, 3.0]], dtype=torch.float64))
    assert p[0].tolist() == pytest.approx([0.09003057, 0.24472847, 0.66524096], abs=1e-7)   # cpu_test.go


def test_rms_norm_hand_values_and_the_plus_one():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.zeros(2), 0.0)                          # w = 0 means scale 1
    assert y[0].tolist() == pytest.approx([3 / math.sqrt(12.5), 4 / math.sqrt(12.5)])
    y = P.rms_norm(x, torch.tensor([1.0, -0.5]), 0.0)
    assert y[0].tolist() == pytest.approx([2 * 3 / math.sqrt(12.5), 0.5 * 4 / math.sqrt(12.5)])
    big_eps = P.rms_norm(x, torch.zeros(2), 12.5)                   # eps is added to the mean, inside the root
    assert big_eps[0].tolist() == pytest.approx([3 / 5.0, 4 / 5.0])


def test_gelu_tanh_hand_values():
    v = torch.tensor([-3.0, -1.0, 0.0, 0.5, 2.0], dtype=torch.float64)
    want = [-0.0036373920817729943, -0.15880800939172324, 0.0, 0.34571400982514394, 1.954597694087775]
    assert P.gelu_tanh(v).tolist() == pytest.approx(want, abs=1e-12)


def test_rope_pairs_halves_and_keeps_norms():
    x = torch.randn(2, 5, 8, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    y = P.rope(x, [0, 1, 2, 3, 4], 10000.0)
    assert torch.allclose(y[:, 0], x[:, 0])                                   # position 0 rotates by nothing
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    # feature i pairs with i + 4: position 1, pair 0 rotates by 1 radian
    a, b = x[0, 1, 0], x[0, 1, 4]
    assert y[0, 1, 0].item() == pytest.approx(a * math.cos(1.0) - b * math.sin(1.0))
    assert y[0, 1, 4].item() == pytest.approx(a * math.sin(1.0) + b * math.cos(1.0))
    # scores depend on the distance only
    q, k = x[0:1], x[1:2]
    s1 = (P.rope(q, [7] * 5, 50.0)[0, 0] * P.rope(k, [4] * 5, 50.0)[0, 0]).sum()
    s2 = (P.rope(q, [103] * 5, 50.0)[0, 0] * P.rope(k, [100] * 5, 50.0)[0, 0]).sum()
    assert s1.item() == pytest.approx(s2.item(), abs=1e-4)


def test_masks():
    full = P.visible(5, None)
    assert full.tolist() == torch.tril(torch.ones(5, 5)).bool().tolist()
    w = P.visible(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True]           # the last 3, itself included
    assert w[1].tolist() == [True, True, False, False, False, False]
    assert torch.equal(P.visible(4, 4), P.visible(4, None)) and torch.equal(P.visible(4, 9), P.visible(4, None))


def test_the_window_and_the_caps_matter(plain_models):
    """In the hot models the window changes logits beyond position `window`, not before; both caps bind."""
    cfg, w = plain_models["A_hot"]
    toks = random_tokens(cfg["vocab_size"], 30, 5)
    ref = P.forward_logits(cfg, w, toks)
    wide = P.forward_logits(dict(cfg, sliding_window=4096), w, toks)
    win = cfg["sliding_window"]
    assert torch.allclose(ref[:win], wide[:win], atol=1e-12) and (ref[win:] - wide[win:]).abs().max() > 1e-3
    assert ref.abs().max() <= cfg["final_logit_softcapping"] and ref.abs().max() > 0.9 * cfg["final_logit_softcapping"]
    nocap = P.forward_logits(dict(cfg, attn_logit_softcapping=0.0), w, toks)
    assert (ref - nocap).abs().max() > 1e-3
    causal = P.forward_logits(cfg, w, toks[:12])
    assert torch.allclose(causal, ref[:12], atol=1e-12)                      # later tokens change nothing before them


def test_float32_follows_float64(plain_models):
    for key in ("A", "B_hot"):
        cfg, w = plain_models[key]
        toks = random_tokens(cfg["vocab_size"], 40, 6)
        a, b = P.forward_logits(cfg, w, toks), P.forward_logits(cfg, w, toks, dtype=torch.float32)
        assert (a - b.double()).abs().max() <= 1e-4 * a.abs().max()


def test_sampler_greedy_ties_and_nucleus():
    l = torch.tensor([1.0, 5.0, 5.0, 2.0])
    assert P.sample_token(l, 0.0, 1.0, 0.3) == 1                              # first maximum wins
    p = [0.1, 0.4, 0.2, 0.3]
    assert P.nucleus(p, 0.65) == [1, 3] and P.nucleus(p, 0.71) == [1, 3, 2] and P.nucleus([0.25] * 4, 0.5) == [0, 1]
    logits = torch.log(torch.tensor(p))
    assert P.sample_token(logits, 1.0, 1.0, 0.05) == 0 and P.sample_token(logits, 1.0, 1.0, 0.45) == 1
    assert P.sample_token(logits, 1.0, 0.65, 0.0) == 1 and P.sample_token(logits, 1.0, 0.65, 0.99) == 3
    cold = P.sample_token(logits, 0.01, 1.0, 0.9)
    assert cold == 1                                                         # a low temperature is nearly greedy


def test_repeat_penalty():
    l = torch.tensor([2.0, -2.0, 1.0, 4.0])
    out = P.apply_repeat_penalty(l, [0, 1, 1, 3], 2.0, 3)                    # the last three: 1, 1, 3
    assert out.tolist() == [2.0, -4.0, 1.0, 2.0]
    assert torch.equal(P.apply_repeat_penalty(l, [0, 1], 1.0, 64), l)


def test_greedy_generation_stops_and_counts(plain_models):
    cfg, w = plain_models["A"]
    out, why = P.greedy_generate(cfg, w, [5, 6, 7], 4)
    assert len(out) == 4 and why == "length"
    stop = out[-1]
    out2, why2 = P.greedy_generate(cfg, w, [5, 6, 7], 4, stop=(stop,))
    assert out2 == out[:out.index(stop)] and why2 == "stop"      # ends at the stop token's first occurrence
