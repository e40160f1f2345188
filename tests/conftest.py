"""Shared fixtures: the two tiny Gemma2 configurations and model folders of random weights.

The configurations differ in every size and option (heads and groups, widths that
are no power of two, layers, vocabulary, eps, window, caps, rotary base).  Each
comes with plain random weights (matrices N(0, 0.02), norms N(0, 0.1)) and as a
"hot" variant whose query/key projections and embedding are scaled up, so that
attention scores reach the score cap and logits reach the final cap: with the
plain weights both caps are far away and a fault in them would not show.
Model folders are written into pytest's temporary directory.
"""
from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TINY_A = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=64, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=128, vocab_size=256,
    rope_theta=10000.0, sliding_window=8, query_pre_attn_scalar=16, attn_logit_softcapping=50.0,
    final_logit_softcapping=30.0, rms_norm_eps=1e-6, max_position_embeddings=512, eos_token_id=1)

TINY_B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=96, num_hidden_layers=3,
    num_attention_heads=6, num_key_value_heads=1, head_dim=32, intermediate_size=320, vocab_size=384,
    rope_theta=50000.0, sliding_window=16, query_pre_attn_scalar=24, attn_logit_softcapping=20.0,
    final_logit_softcapping=15.0, rms_norm_eps=1e-5, max_position_embeddings=640, eos_token_id=[1, 7])

# a head size that the tcgen05 prompt kernel takes (a multiple of 64), a window that cuts inside a tile of keys
TINY_C = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=80, num_hidden_layers=2,
    num_attention_heads=3, num_key_value_heads=1, head_dim=64, intermediate_size=136, vocab_size=300,
    rope_theta=20000.0, sliding_window=40, query_pre_attn_scalar=48, attn_logit_softcapping=30.0,
    final_logit_softcapping=20.0, rms_norm_eps=1e-6, max_position_embeddings=768, eos_token_id=2)

# a window that is a whole number of cache pages (as the real 4096 is): the ring is exactly the window, two pages
# with a page-table entry each, and prompts longer than two rings and decoding across the wrap go through the
# cache's page arithmetic, the decode geometry and the graphs' length buckets together; as many key/value heads as
# query heads, an odd vocabulary
TINY_D = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=72, num_hidden_layers=3,
    num_attention_heads=3, num_key_value_heads=3, head_dim=48, intermediate_size=200, vocab_size=211,
    rope_theta=10000.0, sliding_window=128, query_pre_attn_scalar=48, attn_logit_softcapping=25.0,
    final_logit_softcapping=12.0, rms_norm_eps=1e-6, max_position_embeddings=1024, eos_token_id=3)

TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}

HOT_QK, HOT_EMBED = 20.0, 40.0

# whole-model tolerances, as fractions of the largest reference logit of the comparison
F32_MODEL_TOL = 1e-4
BF16_MODEL_TOL = 2e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def write_tiny(model_dir: str, raw_config: dict, seed: int, hot: bool = False, norms_f32: bool = False) -> None:
    """A model folder of seeded random weights; `hot` scales q/k projections and the embedding."""
    from janis_b200 import build_model
    from janis_b200.weights.loader import random_tensors, write_model_folder
    _, cfg, model = build_model(raw_config)
    tensors = random_tensors(model.tensor_specs(), seed, "cpu")
    for name in list(tensors):
        t = tensors[name]
        if hot and (name.endswith("q_proj.weight") or name.endswith("k_proj.weight")):
            tensors[name] = (t.float() * HOT_QK).to(torch.bfloat16)
        elif hot and name == "model.embed_tokens.weight":
            tensors[name] = (t.float() * HOT_EMBED).to(torch.bfloat16)
        elif norms_f32 and name.endswith("norm.weight"):
            tensors[name] = t.float()
    write_model_folder(model_dir, cfg.to_dict(), tensors, {"seed": str(seed)})


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{'A', 'B', 'C', 'D', 'A_hot', ...} -> folder with config.json and model.safetensors."""
    out = {}
    seed = 11
    for name, cfg in TINY.items():
        for hot in (False, True):
            key = name + ("_hot" if hot else "")
            d = tmp_path_factory.mktemp(f"tiny_{key}")
            write_tiny(str(d), cfg, seed, hot=hot, norms_f32=(name == "B"))
            out[key] = str(d)
            seed += 1
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """Each folder as the plain implementation reads it: key -> (config dict, weights)."""
    from tests.plain import gemma2_plain as P
    return {k: P.load_folder(d) for k, d in model_dirs.items()}


_plain_cache: dict = {}


def plain_logits(plain_models, key: str, tokens) -> torch.Tensor:
    """float64 logits [len, vocab] of the plain implementation, remembered per (model, tokens)."""
    from tests.plain import gemma2_plain as P
    k = (key, tuple(tokens))
    if k not in _plain_cache:
        cfg, w = plain_models[key]
        _plain_cache[k] = P.forward_logits(cfg, w, list(tokens))
    return _plain_cache[k]


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
