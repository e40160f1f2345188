"""The whole model at the layer shapes of Gemma2-2B and Gemma2-27B against the plain implementation.

The tiny configurations of the other tests never reach the code that the real sizes select: head sizes 256
and 128 (the tcgen05 prompt kernel and its tensor-memory layout, the tensor-core decode kernel's head groups),
8 query heads over 4 and 32 over 16 key/value heads, widths of 2304 and 4608 (the register-resident norm
kernels, cluster sizes of the skinny products), a window of 4096 whose ring is 64 pages and really wraps.
Here two-layer models of those shapes (two layers: one windowed, one not) run whole prompts, the last 32
tokens one by one, unequal batches with slots used again, short prompt steps replayed from a graph of their
padded shape, and a prompt fed in pieces, in float32 and in bfloat16.

Cut, to keep the oracle quick: two layers instead of 26 and 46, and a vocabulary of 4,096 instead of 256,000.
Everything else of a layer is the real size.  Weights are random (seeded, drawn on the device), with the query
and key projections and the embedding scaled up so that scores reach the score cap and logits the final cap.
The plain implementation runs on the GPU here, in float64 torch operations: it stays the oracle, it is not the
product path.
"""
from __future__ import annotations

import pytest
import torch

from tests.conftest import HOT_EMBED, HOT_QK, random_tokens
from tests.helpers import assert_logits, run_requests
from tests.plain import gemma2_plain as P

pytestmark = pytest.mark.gpu

VOCAB_CUT = 4096

SHAPE_2B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=2304, num_hidden_layers=2,
    num_attention_heads=8, num_key_value_heads=4, head_dim=256, intermediate_size=9216, vocab_size=VOCAB_CUT,
    rope_theta=10000.0, sliding_window=4096, query_pre_attn_scalar=256, attn_logit_softcapping=50.0,
    final_logit_softcapping=30.0, rms_norm_eps=1e-6, max_position_embeddings=8192, eos_token_id=1)

SHAPE_27B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=4608, num_hidden_layers=2,
    num_attention_heads=32, num_key_value_heads=16, head_dim=128, intermediate_size=36864, vocab_size=VOCAB_CUT,
    rope_theta=10000.0, sliding_window=4096, query_pre_attn_scalar=144, attn_logit_softcapping=50.0,
    final_logit_softcapping=30.0, rms_norm_eps=1e-6, max_position_embeddings=8192, eos_token_id=1)

SHAPES = {"2b": SHAPE_2B, "27b": SHAPE_27B}


class Rig:
    """One configuration: its random tensors (kept on the device in bfloat16, as a folder would hold them), the
    plain model over them in float64, and engines per dtype."""

    def __init__(self, raw):
        from janis_b200.engine.engine import build_model
        from janis_b200.weights.loader import random_tensors
        self.raw = raw
        _, self.cfg, model = build_model(raw)
        t = random_tensors(model.tensor_specs(), 21, "cuda:0")
        for name in list(t):
            if name.endswith("q_proj.weight") or name.endswith("k_proj.weight"):
                t[name] = (t[name].float() * HOT_QK / 4).to(torch.bfloat16)       # wider rows than the tiny models': a smaller factor
            elif name == "model.embed_tokens.weight":
                t[name] = (t[name].float() * HOT_EMBED).to(torch.bfloat16)
        self.tensors = t
        self.plain_w = None
        self._plain: dict = {}

    def engine(self, dtype, **kw):
        from janis_b200.engine.engine import Engine, _dtype, _runtime, build_model
        from janis_b200.parts.base import WeightStore
        _, _, model = build_model(self.raw)
        rt = _runtime(dtype, "cuda:0")
        model.load(WeightStore({k: v.clone() for k, v in self.tensors.items()}), rt)
        return Engine(model, rt, kw.pop("max_tokens", 8192), kw.pop("max_batch", None), None, 16384, kw.pop("use_graphs", True))

    def plain(self, tokens):
        key = tuple(tokens)
        if key not in self._plain:
            if self.plain_w is None:
                self.plain_w = {k: v.double() for k, v in self.tensors.items()}
            self._plain[key] = P.forward_logits(self.cfg.to_dict(), self.plain_w, list(tokens)).cpu()
        return self._plain[key]


@pytest.fixture(scope="module", params=["2b", "27b"])
def rig(request):
    r = Rig(SHAPES[request.param])
    r.name = request.param
    yield r
    r.tensors = r.plain_w = None
    torch.cuda.empty_cache()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_last_32_and_unequal_batches_at_real_layer_shapes(rig, dtype):
    """Requests alone and whole, with their last 32 tokens one by one, and in batches of two whose shorter
    request ends earlier, one batch after another over the same slots.  At the 2B shape one request is longer
    than the window's ring (4,300 tokens: its prompt of 4,268 is attended from the step's own keys, stored as
    its last 4,096, and the 32 tokens that follow wrap the ring)."""
    eng = rig.engine(dtype, max_tokens=2 * 4352, max_batch=2)
    lens = ([4300] if rig.name == "2b" else [700]) + [150, 70, 33, 257]
    reqs = [random_tokens(VOCAB_CUT, n, 2000 + i) for i, n in enumerate(lens)]
    got = run_requests(eng, reqs, [n - 32 for n in lens], max_live=2)
    for i, (g, r) in enumerate(zip(got, reqs)):
        assert_logits(g, rig.plain(r), dtype, f"{rig.name} shape, request {i} of {lens[i]} tokens, last 32 one by one")
    whole = run_requests(eng, reqs[1:3], [150, 70], max_live=1)
    for i, g in enumerate(whole):
        assert_logits(g, rig.plain(reqs[1 + i]), dtype, f"{rig.name} shape, request {1 + i} whole")
    assert eng.cache.live_slots() == []
    eng.cache.audit()
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_graphed_prompt_steps_and_pieces_at_real_layer_shapes(rig, dtype):
    """Short prompt steps of one padded shape, three times (launched, recorded, replayed) with the workspace
    poisoned in between, then tokens over what they stored; and a prompt that comes in pieces of 100 tokens."""
    from janis_b200 import StepEntry
    eng = rig.engine(dtype, max_tokens=4096, max_batch=4)
    for b, lens in enumerate([(30, 75, 12), (41, 50, 33), (64, 60, 3)]):
        reqs = [random_tokens(VOCAB_CUT, n + 2, 2100 + 10 * b + i) for i, n in enumerate(lens)]
        slots = [eng.alloc_slot() for _ in reqs]
        eng.stepper.ws.fill(float("nan"))
        out = eng.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lens)])
        for i, n in enumerate(lens):
            assert_logits(out[i:i + 1], rig.plain(reqs[i])[n - 1:n], dtype, f"{rig.name} shape, batch {b} prompt {i}")
        for t in range(2):
            eng.stepper.ws.fill(float("nan"))
            out = eng.step([StepEntry(s, [r[n + t]], [0]) for s, r, n in zip(slots, reqs, lens)])
            for i, n in enumerate(lens):
                assert_logits(out[i:i + 1], rig.plain(reqs[i])[n + t:n + t + 1], dtype,
                              f"{rig.name} shape, batch {b} request {i} token {t}")
        for s in slots:
            eng.free_slot(s)
    assert len(eng.stepper._prompt_graphs) == 1
    req = random_tokens(VOCAB_CUT, 330, 2200)
    slot = eng.alloc_slot()
    got = []
    for a in range(0, 330, 100):
        piece = req[a:a + 100]
        got.append(eng.step([StepEntry(slot, piece, list(range(len(piece))))]).cpu())
    assert_logits(torch.cat(got), rig.plain(req), dtype, f"{rig.name} shape, a prompt in pieces of 100")
    eng.free_slot(slot)
    eng.cache.audit()
    eng.close()
