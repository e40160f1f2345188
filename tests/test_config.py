"""Configuration and registry: keys, defaults, guards that return errors, registration.
After the reference's `qwen/config_test.go:12-111` and `qwen/config_guard_test.go:17-60`
(a bad config must be an error, never a crash)."""
from __future__ import annotations

import json

import pytest

import janis_b200
from janis_b200.config.base import ConfigError, read_config_json
from janis_b200.config.gemma2 import FULL, SLIDING, Gemma2Config
from tests.conftest import TINY_A, TINY_B


def test_every_key_is_read_from_config_json():
    a, b = Gemma2Config.from_dict(TINY_A), Gemma2Config.from_dict(TINY_B)
    for cfg, raw in ((a, TINY_A), (b, TINY_B)):
        for key in ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
                    "intermediate_size", "vocab_size", "rope_theta", "sliding_window", "query_pre_attn_scalar",
                    "attn_logit_softcapping", "final_logit_softcapping", "rms_norm_eps", "max_position_embeddings"):
            assert getattr(cfg, key) == raw[key], key
    assert a.eos_token_id == (1,) and b.eos_token_id == (1, 7)
    assert a.layer_types == (SLIDING, FULL) and b.layer_types == (SLIDING, FULL, SLIDING)


def test_defaults_of_absent_keys():
    raw = dict(hidden_size=64, num_attention_heads=4, num_hidden_layers=1, vocab_size=10, intermediate_size=16)
    c = Gemma2Config.from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16           # qwen/config.go:196-203
    assert c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.query_pre_attn_scalar == 16.0
    assert c.attn_logit_softcapping == 0.0 and c.final_logit_softcapping == 0.0
    assert c.sliding_window == 4096 and c.max_position_embeddings == 8192
    assert c.tie_word_embeddings is True and c.eos_token_id == ()


def test_layer_types_list_overrides_the_alternation():
    raw = dict(TINY_B, layer_types=[FULL, FULL, SLIDING])
    assert Gemma2Config.from_dict(raw).layer_types == (FULL, FULL, SLIDING)
    with pytest.raises(ConfigError, match="layer_types names 2"):
        Gemma2Config.from_dict(dict(TINY_B, layer_types=[FULL, FULL]))
    with pytest.raises(ConfigError, match="unknown layer type"):
        Gemma2Config.from_dict(dict(TINY_B, layer_types=[FULL, "chunked", FULL]))


def test_round_trip_through_config_json(tmp_path):
    c = Gemma2Config.from_dict(TINY_B)
    (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
    assert Gemma2Config.from_dict(read_config_json(str(tmp_path))) == c


@pytest.mark.parametrize("change,match", [
    (dict(hidden_size=0), "hidden_size"),
    (dict(num_attention_heads=0), "num_attention_heads"),
    (dict(num_hidden_layers=0), "num_hidden_layers"),
    (dict(num_key_value_heads=3), "not divisible"),
    (dict(head_dim=15), "even"),
    (dict(vocab_size=-5), "vocab_size"),
    (dict(intermediate_size="big"), "must be an integer"),
    (dict(rope_theta=0), "rope_theta"),
    (dict(rms_norm_eps=-1e-6), "rms_norm_eps"),
    (dict(query_pre_attn_scalar=0), "query_pre_attn_scalar"),
    (dict(attn_logit_softcapping=-1), "attn_logit_softcapping"),
    (dict(sliding_window=0), "sliding_window"),
    (dict(tie_word_embeddings=False), "tie_word_embeddings"),
    (dict(hidden_activation="relu"), "hidden_activation"),
    (dict(quantization={"group_size": 64, "bits": 4}), "quantized"),
    (dict(eos_token_id="two"), "eos_token_id"),
])
def test_bad_configs_are_errors(change, match):
    with pytest.raises(ConfigError, match=match):
        Gemma2Config.from_dict(dict(TINY_A, **change))


def test_missing_required_key_names_it():
    raw = dict(TINY_A)
    del raw["vocab_size"]
    with pytest.raises(ConfigError, match="vocab_size"):
        Gemma2Config.from_dict(raw)


def test_missing_and_broken_files(tmp_path):
    with pytest.raises(ConfigError, match="read config.json"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="parse config.json"):
        read_config_json(str(tmp_path))
    (tmp_path / "config.json").write_text("[1, 2]")
    with pytest.raises(ConfigError, match="JSON object"):
        read_config_json(str(tmp_path))


def test_registry_resolves_by_architecture_then_model_type():
    assert "Gemma2ForCausalLM" in janis_b200.architectures()
    assert janis_b200.resolve({"architectures": ["Gemma2ForCausalLM"]}).name == "Gemma2ForCausalLM"
    assert janis_b200.resolve({"model_type": "gemma2"}).name == "Gemma2ForCausalLM"
    with pytest.raises(ConfigError, match="unsupported architecture 'LlamaForCausalLM'"):
        janis_b200.resolve({"architectures": ["LlamaForCausalLM"], "model_type": "llama"})
    with pytest.raises(ConfigError, match="unsupported model_type 'whisper'"):
        janis_b200.resolve({"model_type": "whisper"})


def test_registering_twice_needs_replace():
    with pytest.raises(ValueError, match="already registered"):
        janis_b200.register_architecture("Gemma2ForCausalLM", Gemma2Config, lambda c: None)


def test_the_model_is_built_from_the_configuration_alone():
    """Two configurations, two differently sized models, no size from anywhere else."""
    for raw in (TINY_A, TINY_B):
        _, cfg, model = janis_b200.build_model(raw)
        specs = model.tensor_specs()
        H, I, V = raw["hidden_size"], raw["intermediate_size"], raw["vocab_size"]
        nq, nkv, hd = raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"]
        assert specs["model.embed_tokens.weight"].shape == (V, H)
        assert specs["model.layers.0.self_attn.q_proj.weight"].shape == (nq * hd, H)
        assert specs["model.layers.0.self_attn.k_proj.weight"].shape == (nkv * hd, H)
        assert specs["model.layers.0.self_attn.o_proj.weight"].shape == (H, nq * hd)
        assert specs["model.layers.0.mlp.gate_proj.weight"].shape == (I, H)
        assert specs["model.layers.0.mlp.down_proj.weight"].shape == (H, I)
        assert len(specs) == 2 + 11 * raw["num_hidden_layers"]
        needs = model.cache_line_needs()
        assert [n["kv"].window for n in needs] == [raw["sliding_window"] if i % 2 == 0 else None
                                                   for i in range(raw["num_hidden_layers"])]
        blk = model.blocks[0]
        assert blk.mixer.scale == pytest.approx(raw["query_pre_attn_scalar"] ** -0.5)
        assert blk.mixer.softcap == raw["attn_logit_softcapping"] and model.head.softcap == raw["final_logit_softcapping"]
        assert blk.first_norm.eps == raw["rms_norm_eps"] and blk.mixer.position.base == raw["rope_theta"]
