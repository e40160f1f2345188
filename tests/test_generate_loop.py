"""The generation loop's decisions with a fake backend, apart from any model (the reference tests
its session the same way with a fake forward, `qwen/session_pin_test.go:55-129`)."""
from __future__ import annotations

import pytest

from janis_b200.engine.generate import GenerationError, Reply, generate, plan_batches


class FakeBackend:
    """Next token = (last token + 1) % 100; prompts prefill to (last prompt token + 1).  Counts what the
    loop asks of it and checks that places are opened and closed exactly once."""

    def __init__(self, max_batch=4, max_context=64, room=1000):
        self.max_batch, self.max_context, self.room = max_batch, max_context, room
        self.open_handles, self.next_handle = set(), 0
        self.closed = []
        self.prefills, self.decodes = [], []
        self.live_peak = 0
        self.device_tokens, self.in_flight, self.layouts = None, 0, []

    def fits(self, final_lengths):
        return sum(final_lengths) <= self.room

    def open(self):
        h = self.next_handle
        self.next_handle += 1
        self.open_handles.add(h)
        self.live_peak = max(self.live_peak, len(self.open_handles))
        return h

    def close(self, h):
        assert h in self.open_handles, "closed twice or never opened"
        self.open_handles.remove(h)
        self.closed.append(h)

    def prefill(self, handles, prompts, request_ids, banned):
        assert set(handles) <= self.open_handles
        self.prefills.append((list(request_ids), banned))
        out = [(p[-1] + 1) % 100 for p in prompts]
        if banned:
            out = [t if t not in banned else (t + 1) % 100 for t in out]
        return out

    lookahead = False

    def keeps_layout(self, n_live, n_rows):
        return n_live * 2 > n_rows                 # re-form once half the rows are holes

    def decode_start(self, handles, last_tokens, request_ids, token_index, replies):
        live = [h is not None for h in handles]
        assert all(h in self.open_handles for h, ok in zip(handles, live) if ok)
        if last_tokens is None:                    # tokens stay "on the device": the ones of the step before
            assert self.lookahead and self.device_tokens is not None and len(self.device_tokens) == len(handles)
            last_tokens = self.device_tokens
            for idx, r, ok in zip(token_index, replies, live):
                assert not ok or idx == len(r) + 1     # the step before has not been read yet
        else:
            for idx, r, ok in zip(token_index, replies, live):
                assert not ok or idx == len(r)
        self.decodes.append([r for r, ok in zip(request_ids, live) if ok])
        self.layouts.append(list(request_ids))
        out = [(t + 1) % 100 for t in last_tokens]
        self.device_tokens = out
        self.in_flight += 1
        assert self.in_flight <= 2
        return out

    def decode_finish(self, ticket):
        self.in_flight -= 1
        return ticket


class LookaheadBackend(FakeBackend):
    lookahead = True


def test_length_limit_and_order_of_replies():
    b = FakeBackend()
    out = generate(b, [[10], [20, 21], [30]], max_tokens=3)
    assert [r.tokens for r in out] == [[11, 12, 13], [22, 23, 24], [31, 32, 33]]
    assert all(r.finish_reason == "length" for r in out)
    assert len(b.prefills) == 1 and len(b.decodes) == 2            # the last token is not fed back
    assert not b.open_handles and sorted(b.closed) == [0, 1, 2]


def test_stop_token_ends_a_reply_and_is_not_part_of_it():
    b = FakeBackend()
    out = generate(b, [[10], [47]], max_tokens=10, stop=[13, 50])
    assert out[0].tokens == [11, 12] and out[0].finish_reason == "stop"
    assert out[1].tokens == [48, 49] and out[1].finish_reason == "stop"


def test_shorter_requests_leave_the_batch_earlier():
    b = FakeBackend()
    out = generate(b, [[10], [20], [30]], max_tokens=6, stop=[12, 23])
    assert [r.tokens for r in out] == [[11], [21, 22], [31, 32, 33, 34, 35, 36]]
    assert b.decodes[0] == [0, 1, 2] and b.decodes[1] == [1, 2] and all(d == [2] for d in b.decodes[2:])
    assert b.closed[:2] == [0, 1]                                  # places come back as sequences end


def test_first_token_can_be_a_stop():
    b = FakeBackend()
    out = generate(b, [[10]], max_tokens=5, stop=[11])
    assert out[0].tokens == [] and out[0].finish_reason == "stop" and not b.decodes
    b = FakeBackend()
    out = generate(b, [[10]], max_tokens=3, stop=[11], mask_stop_on_first=True)
    assert b.prefills[0][1] == [11] and out[0].tokens == [12, 13, 14]


def test_requests_beyond_one_batch_run_in_later_batches():
    b = FakeBackend(max_batch=2)
    out = generate(b, [[i] for i in range(5)], max_tokens=2)
    assert [r.tokens for r in out] == [[i + 1, i + 2] for i in range(5)]
    assert [p[0] for p in b.prefills] == [[0, 1], [2, 3], [4]] and b.live_peak == 2
    b = FakeBackend(max_batch=8, room=30)                          # room decides: 3 requests of 10 tokens at most
    generate(b, [[1]] * 7, max_tokens=9)
    assert [len(p[0]) for p in b.prefills] == [3, 3, 1]
    with pytest.raises(GenerationError, match="more than the cache holds"):
        generate(FakeBackend(room=5), [[1, 2, 3]], max_tokens=9)


def test_plan_batches_keeps_order():
    assert plan_batches([5, 5, 5, 5], 3, lambda ls: sum(ls) <= 12) == [[0, 1], [2, 3]]
    assert plan_batches([], 3, lambda ls: True) == []


def test_context_is_a_limit_too():
    b = FakeBackend(max_context=8)
    out = generate(b, [[1, 2, 3, 4, 5]], max_tokens=50)
    assert len(out[0].tokens) == 3 and out[0].finish_reason == "length"   # 5 + 3 = 8
    with pytest.raises(GenerationError, match="no room"):
        generate(b, [[0] * 8], max_tokens=5)


def test_empty_prompt_and_default_length():
    b = FakeBackend(max_context=10 ** 6, room=10 ** 9)
    out = generate(b, [[], [5]], max_tokens=0)                     # <= 0 means the reference's default of 512
    assert out[0].tokens == [] and out[0].finish_reason == "empty"
    assert len(out[1].tokens) == 512


def test_callbacks_and_cancel():
    b = FakeBackend(max_batch=2)
    heard = []
    calls = [0]

    def cancel():
        calls[0] += 1
        return calls[0] >= 3

    out = generate(b, [[10], [20], [30]], max_tokens=10, on_token=lambda i, t: heard.append((i, t)), cancel=cancel)
    assert out[0].tokens == [11, 12, 13] and out[1].tokens == [21, 22, 23]
    assert [r.finish_reason for r in out] == ["cancel", "cancel", "cancel"] and out[2].tokens == []
    assert heard == [(0, 11), (1, 21), (0, 12), (1, 22), (0, 13), (1, 23)]
    assert not b.open_handles


def test_places_are_closed_when_the_backend_fails():
    class Broken(FakeBackend):
        def decode_start(self, *a):
            raise RuntimeError("boom")

    b = Broken()
    with pytest.raises(RuntimeError, match="boom"):
        generate(b, [[1], [2]], max_tokens=4)
    assert not b.open_handles


@pytest.mark.parametrize("max_tokens,stop", [(6, ()), (6, (12, 23)), (9, (33, 11, 52)), (1, ()), (3, (21,))])
def test_lookahead_gives_the_same_replies(max_tokens, stop):
    """Starting a step before the one before it has been read changes no reply: ends by length are known
    beforehand, a stop token is seen a step late and the token computed past it is dropped."""
    prompts = [[10], [20], [30], [40, 41], [50]]
    plain = generate(FakeBackend(max_batch=3), prompts, max_tokens=max_tokens, stop=stop)
    b = LookaheadBackend(max_batch=3)
    ahead = generate(b, prompts, max_tokens=max_tokens, stop=stop)
    assert [(r.tokens, r.finish_reason) for r in ahead] == [(r.tokens, r.finish_reason) for r in plain]
    assert not b.open_handles and b.in_flight == 0


def test_lookahead_keeps_rows_in_place_and_reforms_when_half_are_holes():
    b = LookaheadBackend(max_batch=4)
    out = generate(b, [[10], [20], [30], [40]], max_tokens=8, stop=(12, 22, 33))
    assert [r.tokens for r in out] == [[11], [21], [31, 32], [41, 42, 43, 44, 45, 46, 47, 48]]
    # requests 0 and 1 meet their stop token in the first decode step; the second step, started before the
    # first was read, still has their rows.  With two of four rows empty no third step is started ahead:
    # the second is read (request 2 stops there) and the layout is formed anew from what is still open
    assert b.layouts[0] == [0, 1, 2, 3] and b.layouts[1] == [0, 1, 2, 3]
    assert b.layouts[2] == [3] and all(l == [3] for l in b.layouts[2:])


def test_lookahead_and_cancel():
    b = LookaheadBackend(max_batch=2)
    calls = [0]

    def cancel():
        calls[0] += 1
        return calls[0] >= 4

    out = generate(b, [[10], [20], [30]], max_tokens=10, cancel=cancel)
    assert [r.finish_reason for r in out] == ["cancel"] * 3 and out[2].tokens == []
    assert out[0].tokens == [11, 12, 13, 14] and not b.open_handles and b.in_flight == 0


@pytest.mark.parametrize("backend", [FakeBackend, LookaheadBackend])
def test_a_length_limit_for_each_request(backend):
    """`max_tokens` as a list: each reply ends at its own limit (0 stands for the default), the others go on; the
    room a batch needs is planned from each request's own limit."""
    b = backend(max_batch=4, max_context=700)
    out = generate(b, [[10], [20], [30], [40]], max_tokens=[2, 5, 1, 0], stop=())
    assert [len(r.tokens) for r in out] == [2, 5, 1, 512]
    assert out[0].tokens == [11, 12] and out[1].tokens == [21, 22, 23, 24, 25] and out[2].tokens == [31]
    assert all(r.finish_reason == "length" for r in out)
    assert not b.open_handles and sorted(b.closed) == [0, 1, 2, 3]
    # planned from the limits: 1 + 30 and 1 + 3 fit a room of 40 together, 1 + 30 twice do not
    assert plan_batches([31, 4], 4, lambda ls: sum(ls) <= 40) == [[0, 1]]
    b = backend(max_batch=4, room=40)
    generate(b, [[1], [2], [3]], max_tokens=[30, 3, 30], stop=())
    assert [sorted(p[0]) for p in b.prefills] == [[0, 1], [2]]
    with pytest.raises(GenerationError, match="3 token limits for 2 requests"):
        generate(backend(), [[1], [2]], max_tokens=[1, 2, 3])
