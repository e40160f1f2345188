"""Gemma2 as an arrangement of parts.

Everything here comes from the configuration: sizes, the norms' eps, the rotary
base, the score scale 1/sqrt(query_pre_attn_scalar) (`gemma/gemma.go:62`), the
two caps, the window and which layers slide.  Tensor names are the checkpoint's
(`gemma/gemma.go:135-155`, `:179`, `:189`, `:242`), each with `.weight`; the
head is tied to the embedding (`gemma/gemma.go:169-176`, `:210`).
"""
from __future__ import annotations

import math

import numpy as np

from ..config.gemma2 import SLIDING, Gemma2Config
from ..engine.model import DecoderModel, LayerCall
from ..parts import registry as parts
from ..registry import register_architecture


def build_gemma2(cfg: Gemma2Config) -> DecoderModel:
    H, hd = cfg.hidden_size, cfg.head_dim

    def norm(name):
        return parts.make("norm", "rms_norm", width=H, eps=cfg.rms_norm_eps, weight_name=name, offset=1.0)

    blocks = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        mixer = parts.make(
            "mixer", "softmax_attention", hidden=H, n_heads=cfg.num_attention_heads,
            n_kv_heads=cfg.num_key_value_heads, head_dim=hd,
            scale=1.0 / math.sqrt(cfg.query_pre_attn_scalar), softcap=cfg.attn_logit_softcapping,
            window=cfg.sliding_window if cfg.layer_types[i] == SLIDING else None,
            position=parts.make("position", "rotary", head_dim=hd, base=cfg.rope_theta),
            names={k: f"{p}.self_attn.{k}_proj.weight" for k in ("q", "k", "v", "o")})
        ff = parts.make("feed_forward", "gated_mlp", hidden=H, intermediate=cfg.intermediate_size,
                        act=cfg.hidden_activation,
                        names={k: f"{p}.mlp.{k}_proj.weight" for k in ("gate", "up", "down")})
        blocks.append(parts.make(
            "block", "sandwich", mixer=mixer, feed_forward=ff,
            input_norm=norm(f"{p}.input_layernorm.weight"),
            post_mixer_norm=norm(f"{p}.post_attention_layernorm.weight"),
            pre_ff_norm=norm(f"{p}.pre_feedforward_layernorm.weight"),
            post_ff_norm=norm(f"{p}.post_feedforward_layernorm.weight")))
    table = "model.embed_tokens.weight"
    return DecoderModel(
        cfg,
        embedding=parts.make("embedding", "scaled_table", vocab=cfg.vocab_size, hidden=H, table_name=table,
                             scale=float(np.float32(math.sqrt(float(H))))),
        blocks=blocks,
        final_norm=norm("model.norm.weight"),
        head=parts.make("head", "capped_linear", vocab=cfg.vocab_size, hidden=H, table_name=table,
                        softcap=cfg.final_logit_softcapping),
        schedule=[LayerCall(i, i) for i in range(cfg.num_hidden_layers)],
        ignorable_tensors=("lm_head.weight", "*.rotary_emb.inv_freq"),
        stop_tokens=cfg.eos_token_id,
        max_context=cfg.max_position_embeddings)


register_architecture("Gemma2ForCausalLM", Gemma2Config, build_gemma2, model_types=("gemma2",), replace=True)
