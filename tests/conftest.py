"""Shared fixtures: the two tiny Gemma2 configurations and model folders of random weights.

The configurations differ in every size and option (heads and groups, widths that
are no power of two, layers, vocabulary, eps, window, caps, rotary base).  Model
folders are written into pytest's temporary directory.
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

TINY = {"A": TINY_A, "B": TINY_B}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """{'A': folder, 'B': folder} with config.json and model.safetensors (bfloat16, seeds 11 and 12)."""
    import janis_b200
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        janis_b200.write_random_model(str(d), cfg, seed=11 + i)
        out[name] = str(d)
    return out


@pytest.fixture(scope="session")
def plain_models(model_dirs):
    """{'A': (config dict, weights), ...} as the plain implementation reads them."""
    from tests.plain import gemma2_plain as P
    return {k: P.load_folder(d) for k, d in model_dirs.items()}
