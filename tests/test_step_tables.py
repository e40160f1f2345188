"""The host side of a graphed prompt step: how a step's shape is padded and what its tables say about the
padding (no GPU needed)."""
from __future__ import annotations

import numpy as np
import pytest

from janis_b200.engine.step import (StepEntry, Stepper, _bucket_prompt_seqs, _bucket_prompt_tokens, prompt_tables)


def test_padded_shapes():
    sizes = [_bucket_prompt_tokens(n) for n in range(1, Stepper.PROMPT_GRAPH_TOKENS + 1)]
    assert all(b >= n for n, b in zip(range(1, 513), sizes))
    assert sizes == sorted(sizes) and sizes[-1] == Stepper.PROMPT_GRAPH_TOKENS
    assert len(set(sizes)) == 12
    with pytest.raises(ValueError):
        _bucket_prompt_tokens(Stepper.PROMPT_GRAPH_TOKENS + 1)
    # always room for a padding sequence, powers of two
    for n in range(1, Stepper.PROMPT_GRAPH_SEQS):
        b = _bucket_prompt_seqs(n)
        assert b > n and b & (b - 1) == 0 and b <= Stepper.PROMPT_GRAPH_SEQS


def test_tables_of_a_padded_prompt_step():
    Tmax, Smax = 512, 32
    entries = [StepEntry(4, [11, 12, 13], (2,)), StepEntry(0, [21], ()), StepEntry(9, [31, 32, 33, 34, 35], (0, 4))]
    lens = [3, 1, 5]
    Tb = _bucket_prompt_tokens(sum(lens))
    host = prompt_tables(entries, lens, Tb, Tmax, Smax)
    assert host.dtype == np.int32 and host.shape == (3 * Tmax + 5 * Smax,)
    T = 9
    assert host[:T].tolist() == [11, 12, 13, 21, 31, 32, 33, 34, 35] and not host[T:Tmax].any()
    assert host[Tmax:Tmax + T].tolist() == [0, 1, 2, 0, 0, 1, 2, 3, 4]
    assert host[Tmax + T:Tmax + Tb].tolist() == list(range(Tb - T)) and not host[Tmax + Tb:2 * Tmax].any()
    seq = host[2 * Tmax:3 * Tmax]
    assert seq[:T].tolist() == [0, 0, 0, 1, 2, 2, 2, 2, 2]
    assert (seq[T:Tb] == 3).all() and not seq[Tb:].any()        # padding tokens name the first padding sequence
    o = 3 * Tmax
    slots = host[o:o + Smax]
    assert slots[:3].tolist() == [4, 0, 9] and (slots[3:] == -1).all()
    assert not host[o + Smax:o + 2 * Smax].any()                 # every sequence starts at 0
    ends = host[o + 2 * Smax:o + 3 * Smax]
    # the padding tokens are a sequence of their own (every row of the step is some sequence's); the rest hold none
    assert ends[:3].tolist() == lens and ends[3] == Tb - T and not ends[4:].any()
    first = host[o + 3 * Smax:o + 4 * Smax]
    assert first[:3].tolist() == [0, 3, 4] and first[3] == T and (first[4:] == Tb).all()
    # sequences tile the step's rows without a gap
    assert all(first[i] + ends[i] == first[i + 1] for i in range(4))
    rows = host[o + 4 * Smax:o + 5 * Smax]
    assert rows[:3].tolist() == [2, 4, 8] and not rows[3:].any()


def test_tables_of_a_step_that_fills_its_shape():
    entries = [StepEntry(1, list(range(16)), (15,))]
    host = prompt_tables(entries, [16], 16, 512, 32)
    assert (host[2 * 512:2 * 512 + 16] == 0).all() and not host[2 * 512 + 16:3 * 512].any()
    o = 3 * 512
    assert host[o + 2 * 32:o + 2 * 32 + 2].tolist() == [16, 0]       # no padding token: the padding sequence is empty
