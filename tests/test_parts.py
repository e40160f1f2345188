"""Each part alone against the plain implementation's function for it, and the openness of the
arrangement: a toy architecture, defined here, whose layers use a toy mixer with state of its own
(also defined here) beside softmax attention, in pre-norm blocks, with a schedule that names a layer
twice and lets a layer read another layer's keys.  Nothing in the package knows about any of it.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import janis_b200
from janis_b200.cache.cache import KVNeed, ModelCache, StateNeed
from janis_b200.engine.engine import Engine
from janis_b200.engine.model import DecoderModel, LayerCall
from janis_b200.parts import registry as parts
from janis_b200.parts.base import FeedForward, Mixer, PositionEncoding, Runtime, StepContext, WeightStore, Workspace
from janis_b200.parts.embedding import Embedding, LMHead
from janis_b200.weights.loader import TensorSpec, random_tensors
from tests import kernel_refs
from tests.conftest import random_tokens
from tests.helpers import run_in_pieces, run_requests
from tests.plain import gemma2_plain as P

GPU = pytest.mark.gpu
CASES = [pytest.param("cuda", torch.float32, marks=GPU), pytest.param("cuda", torch.bfloat16, marks=GPU),
         pytest.param("refs", torch.float32)]


def runtime(on, dtype):
    if on == "cuda":
        from janis_b200.kernels import ops
        return Runtime(dtype, "cuda:0", ops)
    return Runtime(dtype, "cpu", kernel_refs)


def context(rt, lens, slots=None, mode="prefill"):
    """A prompt step over new sequences of these lengths."""
    n = len(lens)
    dev = rt.device
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    first = [0] + list(np.cumsum(lens)[:-1])
    return StepContext(rt=rt, ws=Workspace(dev), mode=mode, n_tok=sum(lens), n_seq=n,
                       tokens=i32([0] * sum(lens)), tok_pos=i32([p for l in lens for p in range(l)]),
                       tok_seq=i32([s for s, l in enumerate(lens) for _ in range(l)]),
                       seq_slot=i32(slots if slots is not None else list(range(n))), seq_start=i32([0] * n),
                       seq_end=i32(lens), seq_first_row=i32(first), len_bound=max(lens))


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


def close(got, want, dtype, what):
    got, want = got.detach().double().cpu(), want.double()
    scale = want.abs().max().item()
    err = (got - want).abs().max().item()
    assert torch.isfinite(got).all() and err <= tol(dtype) * scale, f"{what}: {err:.3e} vs scale {scale:.3e}"


def loaded(part, rt, seed=1, scale=None):
    t = random_tensors(part.tensor_specs(), seed, "cpu")
    if scale:
        t = {k: (v.float() * scale.get(k.split(".")[0], 1.0)).to(v.dtype) for k, v in t.items()}
    store = WeightStore({k: v.to(rt.device) for k, v in t.items()})
    part.load(store, rt)
    for sub in part.sub_parts():
        sub.load(store, rt)
    return {k: v.double() for k, v in t.items()}


@pytest.mark.parametrize("on,dtype", CASES)
def test_rms_norm_part(on, dtype):
    rt = runtime(on, dtype)
    ctx = context(rt, [3, 4])
    H = 96
    n1 = parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name="n1.weight", offset=1.0)
    n2 = parts.make("norm", "rms_norm", width=H, eps=1e-6, weight_name="n2.weight", offset=0.0)
    w1, w2 = loaded(n1, rt)["n1.weight"], loaded(n2, rt, 2)["n2.weight"]
    g = torch.Generator().manual_seed(3)
    h0, r = torch.randn(7, H, generator=g) * 2, (torch.randn(7, H, generator=g)).to(dtype)
    out = torch.empty(7, H, dtype=dtype, device=rt.device)
    n1.forward(h0.to(rt.device), ctx, out)
    close(out, P.rms_norm(h0.double(), w1, 1e-5), dtype, "norm")
    h = h0.clone().to(rt.device)
    y = n1.residual_add(h, r.to(rt.device), ctx, n2, out)
    h_ref = h0.double() + P.rms_norm(r.double(), w1, 1e-5)
    close(h, h_ref, torch.float32, "residual sum")
    close(y, P.rms_norm(h_ref, w2 - 1.0, 1e-6), dtype, "next norm (offset 0: plain weight)")


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("window", [None, 5])
def test_attention_part_over_whole_prompts(on, dtype, window):
    rt = runtime(on, dtype)
    H, nq, nkv, hd = 96, 6, 2, 32
    att = parts.make("mixer", "softmax_attention", hidden=H, n_heads=nq, n_kv_heads=nkv, head_dim=hd,
                     scale=1.0 / math.sqrt(24.0), softcap=20.0, window=window,
                     position=parts.make("position", "rotary", head_dim=hd, base=50000.0),
                     names={k: f"{k}.weight" for k in "qkvo"})
    w = loaded(att, rt, 4, scale={"q": 8.0, "k": 8.0})
    lens = [9, 1, 30]
    ctx = context(rt, lens)
    cache = ModelCache([att.cache_needs()], 8 * 64, 512, dtype, rt.device)
    for s, n in enumerate(lens):
        assert cache.alloc_slot() == s
        cache.reserve(s, n)
    cache.sync()
    x = torch.randn(sum(lens), H, generator=torch.Generator().manual_seed(5)).to(dtype)
    out = att.forward(x.to(rt.device), ctx, cache.line(0))
    o = 0
    for n in lens:
        want = P.attention(x[o:o + n].double(), w["q.weight"], w["k.weight"], w["v.weight"], w["o.weight"], nq, nkv, hd,
                           50000.0, 24.0, 20.0, window)
        close(out[o:o + n], want, dtype, f"attention, sequence of {n}")
        o += n
    # what it left in the cache: rotated keys and plain values of the last sequence
    line = cache.line(0)["kv"]
    k_ref = P.rope((x[10:].double() @ w["k.weight"].T).view(30, nkv, hd).transpose(0, 1), list(range(30)), 50000.0)
    page = int(line.group.table_host[2, 0])
    close(line.k[page, :, :30], k_ref, dtype, "cached keys")
    close(line.v[page, :, :30], (x[10:].double() @ w["v.weight"].T).view(30, nkv, hd).transpose(0, 1), dtype, "cached values")


@pytest.mark.parametrize("on,dtype", CASES)
@pytest.mark.parametrize("T", [5, 70])
def test_gated_mlp_part(on, dtype, T):
    rt = runtime(on, dtype)
    H, I = 96, 320
    ff = parts.make("feed_forward", "gated_mlp", hidden=H, intermediate=I, act="gelu_pytorch_tanh",
                    names={k: f"{k}.weight" for k in ("gate", "up", "down")})
    w = loaded(ff, rt, 6, scale={"gate": 10.0})
    ctx = context(rt, [T])
    x = torch.randn(T, H, generator=torch.Generator().manual_seed(7)).to(dtype)
    out = ff.forward(x.to(rt.device), ctx)
    close(out, P.geglu_mlp(x.double(), w["gate.weight"], w["up.weight"], w["down.weight"]), dtype, "gated mlp")


@pytest.mark.parametrize("on,dtype", CASES)
def test_embedding_and_head_parts(on, dtype):
    rt = runtime(on, dtype)
    V, H = 384, 96
    emb = Embedding(V, H, "table", scale=float(np.float32(math.sqrt(H))))
    head = LMHead(V, H, "table", softcap=15.0)
    t = loaded(emb, rt, 8)["table"]
    head.table = emb.table
    ctx = context(rt, [6])
    toks = torch.tensor([0, 383, 5, 5, 17, 200], dtype=torch.int32, device=rt.device)
    h = torch.empty(6, H, dtype=torch.float32, device=rt.device)
    emb.forward(toks, ctx, h)
    # in bfloat16 the scale is rounded to bfloat16 before the multiply, as the reference's bfloat16 path does
    ratio = float(torch.tensor(emb.scale, dtype=torch.float32).to(dtype)) / emb.scale
    close(h, P.embed(toks.tolist(), t, H) * ratio, torch.float32, "embedding")
    y = (torch.randn(70, H, generator=torch.Generator().manual_seed(9)) * 30).to(dtype)
    out = torch.empty(70, V, dtype=torch.float32, device=rt.device)
    head.forward(y.to(rt.device), ctx, out)
    close(out, 15.0 * torch.tanh(y.double() @ t.T / 15.0), torch.float32 if dtype == torch.float32 else dtype, "head")


@pytest.mark.parametrize("on,dtype", CASES)
def test_sandwich_block_part(on, dtype, plain_models):
    """One Gemma2 block built by the architecture's builder, run alone on a packed prompt step."""
    rt = runtime(on, dtype)
    cfg, w = plain_models["B_hot"]
    _, typed, model = janis_b200.build_model(cfg)
    model.load(WeightStore({k: v.to(torch.bfloat16).to(rt.device) if v.dim() == 2 else v.float().to(rt.device)
                            for k, v in w.items()}), rt)
    lens = [20, 3]
    ctx = context(rt, lens)
    cache = ModelCache(model.cache_line_needs(), 4 * 64, 512, dtype, rt.device)
    for s, n in enumerate(lens):
        cache.alloc_slot()
        cache.reserve(s, n)
    cache.sync()
    h0 = torch.randn(23, typed.hidden_size, generator=torch.Generator().manual_seed(10)) * 3
    for layer in (0, 1):
        h = h0.clone().to(rt.device)
        nxt = model.blocks[2].first_norm
        h, y = model.blocks[layer].forward(h, ctx, cache.line(layer), next_norm=nxt)
        want = torch.cat([P.block(h0[:20].double(), w, layer, cfg), P.block(h0[20:].double(), w, layer, cfg)])
        close(h, want, dtype, f"block {layer}")
        close(y, P.rms_norm(want, w["model.layers.2.input_layernorm.weight"], cfg["rms_norm_eps"]), dtype, "fused next norm")


# ---------------------------------------------------------------------------
# a toy architecture with a toy mixer, defined here
# ---------------------------------------------------------------------------

class RunningMean(Mixer):
    """y_t = W mean(x_0 .. x_t).  State per sequence: the sum of its inputs so far (the count is the
    position).  Written with torch operations: it is a test's part, not the library's."""

    graph_safe = False          # boolean indexing synchronises: the engine then skips CUDA graphs

    def __init__(self, hidden, name):
        self.hidden, self.name = hidden, name

    def tensor_specs(self):
        return {self.name: TensorSpec((self.hidden, self.hidden), init_std=0.1)}

    def cache_needs(self):
        return {"sum": StateNeed((self.hidden,), torch.float32)}

    def load(self, store, rt):
        self.w = store.get(self.name).float()

    def forward(self, x, ctx, line):
        state = line["sum"].data                                   # [slots, hidden]
        seq = ctx.tok_seq[:ctx.n_tok].long()
        slot = ctx.seq_slot[:ctx.n_seq].long()
        live = slot >= 0
        xf = x.float()
        csum = torch.cumsum(xf, dim=0)
        first = ctx.seq_first_row[:ctx.n_seq].long()
        before = torch.where(first > 0, csum[(first - 1).clamp(min=0)].T, torch.zeros_like(first, dtype=torch.float32)).T
        within = csum - before[seq]                                # running sum inside each sequence
        total = within + state[slot.clamp(min=0)][seq]
        if line.write:
            last = (torch.cat([first[1:], torch.tensor([ctx.n_tok], device=first.device)]) - 1)
            state[slot[live]] = total[last[live]]
        y = total / (ctx.tok_pos[:ctx.n_tok].float() + 1.0)[:, None]
        return (y @ self.w.T).to(ctx.rt.dtype)


class RunningMeanInGraphs(RunningMean):
    """The same mixer written so that a step can be recorded into a CUDA graph: no indexing by a mask (which
    synchronises), no host-side shapes that depend on the data.  Sequences meet the state through a 0/1 matrix
    [sequences, slots]; a padding sequence (slot -1) has a row of zeros there: it reads a state of zeros, stores
    nothing and changes no other row, which is what a recorded step asks of every part."""

    graph_safe = True

    def forward(self, x, ctx, line):
        state = line["sum"].data                                   # [slots, hidden]
        T, S = ctx.n_tok, ctx.n_seq
        seq = ctx.tok_seq[:T].long()
        slot = ctx.seq_slot[:S].long()
        own = (slot[:, None] == torch.arange(state.shape[0], device=slot.device)[None, :]).float()     # [S, slots]
        xf = x.float()
        member = (seq[None, :] == torch.arange(S, device=seq.device)[:, None]).float()                 # [S, T]
        rows = torch.arange(T, device=seq.device)
        earlier = (rows[None, :] <= rows[:, None]).float() * member[seq]                                # [T, T]: same sequence, not later
        total = earlier @ xf + (own @ state)[seq]
        if line.write:
            state += own.T @ (member @ xf)                         # every sequence's sum of this step onto its slot
        y = total / (ctx.tok_pos[:T].float() + 1.0)[:, None]
        return (y @ self.w.T).to(ctx.rt.dtype)


@dataclass(frozen=True)
class ToyConfig:
    hidden: int
    vocab: int
    kinds: tuple            # per layer: "mean" or "attn"
    schedule: tuple         # (layer, cache line, write)
    heads: int = 2
    head_dim: int = 16
    intermediate: int = 48

    @classmethod
    def from_dict(cls, raw, where="config.json"):
        return cls(raw["hidden"], raw["vocab"], tuple(raw["kinds"]), tuple(tuple(s) for s in raw["schedule"]),
                   raw.get("heads", 2), raw.get("head_dim", 16), raw.get("intermediate", 48))

    def to_dict(self):
        return {"architectures": ["ToyForCausalLM"], "hidden": self.hidden, "vocab": self.vocab,
                "kinds": list(self.kinds), "schedule": [list(s) for s in self.schedule], "heads": self.heads,
                "head_dim": self.head_dim, "intermediate": self.intermediate}


def build_toy(cfg: ToyConfig) -> DecoderModel:
    H = cfg.hidden
    blocks = []
    for i, kind in enumerate(cfg.kinds):
        if kind == "mean":
            mixer = parts.make("mixer", "test_running_mean", hidden=H, name=f"l{i}.mean.weight")
        else:
            mixer = parts.make("mixer", "softmax_attention", hidden=H, n_heads=cfg.heads, n_kv_heads=1,
                               head_dim=cfg.head_dim, scale=cfg.head_dim ** -0.5,
                               position=parts.make("position", "rotary", head_dim=cfg.head_dim, base=100.0,
                                                   rotary_dims=cfg.head_dim // 2),
                               names={k: f"l{i}.{k}.weight" for k in "qkvo"})
        ff = parts.make("feed_forward", "gated_mlp", hidden=H, intermediate=cfg.intermediate, act="silu",
                        names={k: f"l{i}.{k}.weight" for k in ("gate", "up", "down")})
        blocks.append(parts.make("block", "pre_norm", mixer=mixer, feed_forward=ff,
                                 input_norm=parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name=f"l{i}.n1.weight"),
                                 pre_ff_norm=parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name=f"l{i}.n2.weight")))
    return DecoderModel(cfg, Embedding(cfg.vocab, H, "emb.weight", init_std=1.0), blocks,
                        parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name="final.weight"),
                        LMHead(cfg.vocab, H, "head.weight", init_std=0.3),
                        schedule=[LayerCall(*s) for s in cfg.schedule], max_context=512)


def toy_plain(cfg: ToyConfig, w, ids):
    """The toy model over one whole sequence, in float64, straight from its definition."""
    def norm(x, name):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w[name]        # offset 0

    def rope_half(x, n):                                                              # rotate the first half of each head
        r = cfg.head_dim // 2
        return torch.cat([P.rope(x[..., :r], list(range(n)), 100.0), x[..., r:]], dim=-1)

    n = len(ids)
    h = w["emb.weight"][ids]
    kv = {}
    for layer, line, write in cfg.schedule:
        p = f"l{layer}."
        x = norm(h, p + "n1.weight")
        if cfg.kinds[layer] == "mean":
            y = torch.cumsum(x, 0) / torch.arange(1, n + 1, dtype=torch.float64)[:, None]
            r = y @ w[p + "mean.weight"].T
        else:
            q = rope_half((x @ w[p + "q.weight"].T).view(n, cfg.heads, cfg.head_dim).transpose(0, 1), n)
            if write:
                k = rope_half((x @ w[p + "k.weight"].T).view(n, 1, cfg.head_dim).transpose(0, 1), n)
                v = (x @ w[p + "v.weight"].T).view(n, 1, cfg.head_dim).transpose(0, 1)
                kv[line] = (k, v)
            k, v = kv[line]
            s = (q @ k.transpose(1, 2)) * cfg.head_dim ** -0.5
            s = s.masked_fill(~P.visible(n, None), float("-inf"))
            r = (torch.softmax(s, -1) @ v).transpose(0, 1).reshape(n, -1) @ w[p + "o.weight"].T
        h = h + r
        x = norm(h, p + "n2.weight")
        g = x @ w[p + "gate.weight"].T
        h = h + ((g / (1 + torch.exp(-g))) * (x @ w[p + "up.weight"].T)) @ w[p + "down.weight"].T
    return norm(h, "final.weight") @ w["head.weight"].T


TOY = dict(architectures=["ToyForCausalLM"], hidden=32, vocab=50, kinds=["mean", "attn", "attn", "mean"],
           # layer 1 runs twice (its second visit has a cache line of its own); layer 2 reads layer 1's first keys
           schedule=[[0, 0, True], [1, 1, True], [2, 1, False], [3, 2, True], [1, 3, True]])


@pytest.fixture
def toy_registered():
    parts.register("mixer", "test_running_mean", RunningMean, replace=True)
    janis_b200.register_architecture("ToyForCausalLM", ToyConfig, build_toy, replace=True)
    yield
    parts.unregister("mixer", "test_running_mean")
    janis_b200.unregister_architecture("ToyForCausalLM")


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_toy_architecture_with_a_stateful_mixer(on, dtype, toy_registered):
    rt = runtime(on, dtype)
    arch, cfg, model = janis_b200.build_model(TOY)
    assert arch.name == "ToyForCausalLM" and model.n_cache_lines == 4
    needs = model.cache_line_needs()
    assert isinstance(needs[0]["sum"], StateNeed) and isinstance(needs[1]["kv"], KVNeed) and "sum" in needs[2]
    host = random_tensors(model.tensor_specs(), 21, "cpu")
    model.load(WeightStore({k: v.to(rt.device) for k, v in host.items()}), rt)
    eng = Engine(model, rt, max_tokens=8 * 64, max_batch=3)
    assert eng.stepper.use_graphs is False
    w = {k: v.double() for k, v in host.items()}
    reqs = [random_tokens(50, n, 30 + n) for n in (7, 1, 20, 70, 12)]
    got = run_requests(eng, reqs, [3, 1, 20, 40, 2], max_live=3)       # two batches: slots and state are used again
    for i, (g, r) in enumerate(zip(got, reqs)):
        want = toy_plain(cfg, w, r)
        scale = want.abs().max().item()
        err = (g.double() - want).abs().max().item()
        assert err <= (1e-4 if dtype == torch.float32 else 3e-2) * scale, f"toy request {i}: {err:.3e} / {scale:.3e}"
    # the same requests as prompts that come in pieces of 6 tokens: the stateful mixer goes on from its state, the
    # layer that reads another layer's keys finds that line as the step found it (its writer stores after the last layer)
    for i, (g, r) in enumerate(zip(run_in_pieces(eng, reqs[2:], 6), reqs[2:])):
        want = toy_plain(cfg, w, r)
        scale = want.abs().max().item()
        err = (g.double() - want).abs().max().item()
        assert err <= (1e-4 if dtype == torch.float32 else 3e-2) * scale, f"toy request {i} in pieces: {err:.3e} / {scale:.3e}"
    out = eng.generate([[1, 2, 3], [4]], max_tokens=5, stop=())
    assert [len(o) for o in out] == [5, 5]
    eng.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_stateful_mixer_inside_recorded_steps(dtype):
    """Fixed-size state meets CUDA graphs: the toy architecture with the graph-safe form of its stateful mixer runs its
    decode steps (with padding rows) and its short prompt steps (with padding tokens and sequences) from recorded
    graphs, and gives what it gives launched kernel by kernel, and what the plain model gives."""
    parts.register("mixer", "test_running_mean", RunningMeanInGraphs, replace=True)
    janis_b200.register_architecture("ToyForCausalLM", ToyConfig, build_toy, replace=True)
    try:
        rt = runtime("cuda", dtype)
        outs = []
        host = None
        for graphs in (True, False):
            arch, cfg, model = janis_b200.build_model(TOY)
            assert model.graph_safe
            host = random_tensors(model.tensor_specs(), 21, "cpu")
            model.load(WeightStore({k: v.to(rt.device) for k, v in host.items()}), rt)
            eng = Engine(model, rt, max_tokens=16 * 64, max_batch=5, use_graphs=graphs)
            assert eng.stepper.use_graphs is graphs
            reqs = [random_tokens(50, n, 230 + n) for n in (7, 1, 20, 70, 12)]
            got = None
            for _ in range(3):              # the same shapes three times: launched, recorded, replayed; slots and state used again
                got = run_requests(eng, reqs, [3, 1, 20, 40, 2], max_live=5)
            # prompt steps that ask for the last logits only are recorded once their padded shape has come twice
            from janis_b200 import StepEntry
            last = None
            for _ in range(3):
                slots = [eng.alloc_slot() for _ in reqs[:3]]
                last = eng.step([StepEntry(sl, r, [len(r) - 1]) for sl, r in zip(slots, reqs[:3])]).cpu()
                for sl in slots:
                    eng.free_slot(sl)
            if graphs:
                assert eng.stepper._graphs and eng.stepper._prompt_graphs
            outs.append(got + [last])
            eng.close()
        w = {k: v.double() for k, v in host.items()}
        ends = torch.stack([toy_plain(cfg, w, r)[-1] for r in reqs[:3]])
        for g, how in ((outs[0][-1], "recorded"), (outs[1][-1], "launched")):
            err = (g.double() - ends).abs().max().item()
            assert err <= (1e-4 if dtype == torch.float32 else 3e-2) * ends.abs().max().item(), f"toy prompt step, {how}: {err:.3e}"
        for i, (a, b, r) in enumerate(zip(outs[0][:-1], outs[1][:-1], reqs)):
            want = toy_plain(cfg, w, r)
            scale = want.abs().max().item()
            for g, how in ((a, "recorded"), (b, "launched")):
                err = (g.double() - want).abs().max().item()
                assert err <= (1e-4 if dtype == torch.float32 else 3e-2) * scale, f"toy request {i}, {how}: {err:.3e} / {scale:.3e}"
    finally:
        parts.unregister("mixer", "test_running_mean")
        janis_b200.unregister_architecture("ToyForCausalLM")


# ---------------------------------------------------------------------------
# a feed-forward with routing and another position encoding, defined here and registered
# ---------------------------------------------------------------------------

class Top1Experts(FeedForward):
    """A router picks one of several gated feed-forwards per token (router logits in float32, lowest id on a tie)."""

    def __init__(self, hidden, intermediate, n_experts, prefix):
        self.router_name = prefix + "router.weight"
        self.hidden, self.n_experts = hidden, n_experts
        self.experts = [parts.make("feed_forward", "gated_mlp", hidden=hidden, intermediate=intermediate, act="silu",
                                   names={k: f"{prefix}e{e}.{k}.weight" for k in ("gate", "up", "down")})
                        for e in range(n_experts)]

    def sub_parts(self):
        return list(self.experts)

    def tensor_specs(self):
        return {self.router_name: TensorSpec((self.n_experts, self.hidden), init_std=1.0)}

    def load(self, store, rt):
        self.router = store.get(self.router_name).float()

    def forward(self, x, ctx):
        choice = (x.float() @ self.router.T).argmax(-1)
        out = None
        for e, expert in enumerate(self.experts):
            y = expert.forward(x, ctx)                              # the experts share workspace buffers: take a copy
            y = torch.where((choice == e)[:, None], y, torch.zeros_like(y))
            out = y if out is None else out + y
        return out


class TablePosition(PositionEncoding):
    """A learned row per position added to queries and keys; nothing rotates."""

    def __init__(self, head_dim, max_pos, name):
        self.head_dim, self.max_pos, self.name = head_dim, max_pos, name

    def tensor_specs(self):
        return {self.name: TensorSpec((self.max_pos, self.head_dim), init_std=0.5)}

    def load(self, store, rt):
        self.table = store.get(self.name, rt.dtype)

    def encode(self, qkv, ctx, nq, nkv, hd, with_keys):
        # `encode` alone: storing is the base class's (encode, then the plain store of keys and values), and a
        # prompt that comes in pieces calls `encode` by itself and stores after it has attended
        add = self.table[ctx.tok_pos[:ctx.n_tok].long()]            # [T, hd]
        qkv[:, :(nq + nkv if with_keys else nq)] += add[:, None, :]
        return qkv


@dataclass(frozen=True)
class Toy2Config:
    hidden: int
    vocab: int
    layers: int
    heads: int = 3
    head_dim: int = 16
    intermediate: int = 40
    experts: int = 3

    @classmethod
    def from_dict(cls, raw, where="config.json"):
        return cls(raw["hidden"], raw["vocab"], raw["layers"])

    def to_dict(self):
        return {"architectures": ["Toy2ForCausalLM"], "hidden": self.hidden, "vocab": self.vocab, "layers": self.layers}


def build_toy2(cfg: Toy2Config) -> DecoderModel:
    H = cfg.hidden
    blocks = []
    for i in range(cfg.layers):
        mixer = parts.make("mixer", "softmax_attention", hidden=H, n_heads=cfg.heads, n_kv_heads=1, head_dim=cfg.head_dim,
                           scale=cfg.head_dim ** -0.5,
                           position=parts.make("position", "test_table", head_dim=cfg.head_dim, max_pos=256,
                                               name=f"l{i}.pos.weight"),
                           names={k: f"l{i}.{k}.weight" for k in "qkvo"})
        ff = parts.make("feed_forward", "test_top1", hidden=H, intermediate=cfg.intermediate, n_experts=cfg.experts,
                        prefix=f"l{i}.")
        blocks.append(parts.make("block", "pre_norm", mixer=mixer, feed_forward=ff,
                                 input_norm=parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name=f"l{i}.n1.weight"),
                                 pre_ff_norm=parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name=f"l{i}.n2.weight")))
    return DecoderModel(cfg, Embedding(cfg.vocab, H, "emb.weight", init_std=1.0), blocks,
                        parts.make("norm", "rms_norm", width=H, eps=1e-5, weight_name="final.weight"),
                        LMHead(cfg.vocab, H, "head.weight", init_std=0.3), max_context=256)


def toy2_plain(cfg: Toy2Config, w, ids):
    def norm(x, name):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w[name]

    n = len(ids)
    h = w["emb.weight"][ids]
    margin = float("inf")                        # the smallest gap between the two best router logits
    for i in range(cfg.layers):
        p = f"l{i}."
        x = norm(h, p + "n1.weight")
        t = w[p + "pos.weight"][:n]
        q = (x @ w[p + "q.weight"].T).view(n, cfg.heads, cfg.head_dim) + t[:, None, :]
        k = (x @ w[p + "k.weight"].T).view(n, 1, cfg.head_dim) + t[:, None, :]
        v = (x @ w[p + "v.weight"].T).view(n, 1, cfg.head_dim)
        s = (q.transpose(0, 1) @ k.transpose(0, 1).transpose(1, 2)) * cfg.head_dim ** -0.5
        s = s.masked_fill(~P.visible(n, None), float("-inf"))
        h = h + (torch.softmax(s, -1) @ v.transpose(0, 1)).transpose(0, 1).reshape(n, -1) @ w[p + "o.weight"].T
        x = norm(h, p + "n2.weight")
        logits = x @ w[p + "router.weight"].T
        top = logits.topk(2, dim=-1).values
        margin = min(margin, float((top[:, 0] - top[:, 1]).min()))
        choice = logits.argmax(-1)
        r = torch.zeros_like(h)
        for e in range(cfg.experts):
            g = x @ w[f"{p}e{e}.gate.weight"].T
            y = ((g / (1 + torch.exp(-g))) * (x @ w[f"{p}e{e}.up.weight"].T)) @ w[f"{p}e{e}.down.weight"].T
            r = r + torch.where((choice == e)[:, None], y, torch.zeros_like(y))
        h = h + r
    return norm(h, "final.weight") @ w["head.weight"].T, margin


@pytest.fixture
def toy2_registered():
    parts.register("feed_forward", "test_top1", Top1Experts, replace=True)
    parts.register("position", "test_table", TablePosition, replace=True)
    janis_b200.register_architecture("Toy2ForCausalLM", Toy2Config, build_toy2, replace=True)
    yield
    parts.unregister("feed_forward", "test_top1")
    parts.unregister("position", "test_table")
    janis_b200.unregister_architecture("Toy2ForCausalLM")


@pytest.mark.parametrize("on,dtype", CASES)
def test_a_toy_architecture_with_routing_and_a_position_table(on, dtype, toy2_registered):
    """Routing is a discrete choice: the comparison with the plain model is made in 32-bit, where a router
    logit cannot fall the other way (requests whose closest call is within 1e-3 are left out); in bfloat16
    the model is only run, cached against whole."""
    rt = runtime(on, dtype)
    arch, cfg, model = janis_b200.build_model(dict(architectures=["Toy2ForCausalLM"], hidden=24, vocab=40, layers=2))
    host = random_tensors(model.tensor_specs(), 33, "cpu")
    assert any(k.endswith("router.weight") for k in host) and any(k.endswith("e2.down.weight") for k in host)
    model.load(WeightStore({k: v.to(rt.device) for k, v in host.items()}), rt)
    eng = Engine(model, rt, max_tokens=8 * 64, max_batch=3)
    w = {k: v.double() for k, v in host.items()}
    reqs = [random_tokens(40, n, 60 + n) for n in (9, 1, 33, 70, 12)]
    got = run_requests(eng, reqs, [4, 1, 33, 50, 2], max_live=3)
    checked = 0
    for i, (g, r) in enumerate(zip(got, reqs)):
        assert torch.isfinite(g).all()
        if dtype != torch.float32:
            continue
        want, margin = toy2_plain(cfg, w, r)
        if margin < 1e-3:
            continue
        checked += 1
        scale = want.abs().max().item()
        err = (g.double() - want).abs().max().item()
        assert err <= 1e-4 * scale, f"toy2 request {i}: {err:.3e} / {scale:.3e}"
    assert dtype != torch.float32 or checked >= 3
    # prompts in pieces of 9 tokens equal the same prompts whole (the position table through `encode` alone)
    # (in bfloat16 a router logit may fall the other way between the two ways of running: only run there)
    for i, (g, whole) in enumerate(zip(run_in_pieces(eng, reqs[2:4], 9), got[2:4])):
        assert torch.isfinite(g).all()
        err = (g.double() - whole.double()).abs().max().item()
        assert dtype != torch.float32 or err <= 1e-4 * whole.abs().max().item(), f"toy2 request {i} in pieces"
    out = eng.generate([[1, 2, 3], [4]], max_tokens=4, stop=())
    assert [len(o) for o in out] == [4, 4]
    eng.close()


def test_schedules_are_checked():
    from janis_b200.config.gemma2 import Gemma2Config
    from tests.conftest import TINY_A
    _, cfg, model = janis_b200.build_model(TINY_A)
    blocks = model.blocks
    mk = lambda sched: DecoderModel(cfg, model.embedding, blocks, model.final_norm, model.head, schedule=sched)
    with pytest.raises(ValueError, match="names layer 5"):
        mk([LayerCall(5, 0)])
    with pytest.raises(ValueError, match="written by schedule entries 0 and 1"):
        mk([LayerCall(0, 0), LayerCall(0, 0)])
    with pytest.raises(ValueError, match="before it is written"):
        mk([LayerCall(0, 0, False)])
    with pytest.raises(ValueError, match="keeps something else"):
        mk([LayerCall(0, 0), LayerCall(1, 0, False)])          # a global layer cannot read a window's ring
    with pytest.raises(ValueError, match="never written"):
        mk([LayerCall(0, 1)])
    assert mk([LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2)]).n_cache_lines == 3
