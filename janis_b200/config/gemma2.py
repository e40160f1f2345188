"""Gemma2's configuration: the keys of its config.json, typed.

Keys, defaults and guards follow the reference's parser where it reads them
(`qwen/config.go:81-96`, `:184-237`, `:252-261`).  The reference reads no
`sliding_window` (its Gemma2 leaves the window out, `gemma/gemma.go:7-9`); here
it is read, together with the optional `layer_types` list that names each
layer's kind.  Without that list even layers slide and odd layers see all keys.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Any, Mapping

from .base import ConfigError, ConfigReader

SLIDING = "sliding_attention"
FULL = "full_attention"


@dataclass(frozen=True)
class Gemma2Config:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    intermediate_size: int
    rope_theta: float
    rms_norm_eps: float
    query_pre_attn_scalar: float
    attn_logit_softcapping: float      # 0 = no cap
    final_logit_softcapping: float     # 0 = no cap
    sliding_window: int
    max_position_embeddings: int
    layer_types: tuple[str, ...]       # one of SLIDING / FULL per layer
    eos_token_id: tuple[int, ...] = ()
    tie_word_embeddings: bool = True
    hidden_activation: str = "gelu_pytorch_tanh"
    model_type: str = "gemma2"
    architectures: tuple[str, ...] = ("Gemma2ForCausalLM",)
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str = "config.json") -> "Gemma2Config":
        r = ConfigReader(raw, where)
        if r.has("quantization") or r.has("quantization_config"):
            raise ConfigError(f"{where}: quantized checkpoints are not supported by this engine")
        hidden = r.integer("hidden_size", minimum=1)
        heads = r.integer("num_attention_heads", minimum=1)
        layers = r.integer("num_hidden_layers", minimum=1)
        kv = r.integer("num_key_value_heads", default=heads, minimum=1)     # qwen/config.go:200-203
        if r.has("head_dim"):
            head_dim = r.integer("head_dim", minimum=1)
        else:                                                              # qwen/config.go:196-199
            if hidden % heads:
                raise ConfigError(f"{where}: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        if heads % kv:
            raise ConfigError(f"{where}: num_attention_heads ({heads}) not divisible by "
                              f"num_key_value_heads ({kv})")
        if head_dim % 2:
            raise ConfigError(f"{where}: head_dim must be even for rotary encoding, found {head_dim}")
        window = r.integer("sliding_window", default=4096, minimum=1)
        kinds = r.string_list("layer_types", default=None)
        if kinds:
            if len(kinds) != layers:
                raise ConfigError(f"{where}: layer_types names {len(kinds)} layers, "
                                  f"num_hidden_layers is {layers}")
            for k in kinds:
                if k not in (SLIDING, FULL):
                    raise ConfigError(f"{where}: unknown layer type {k!r} in layer_types")
        else:
            kinds = tuple(SLIDING if i % 2 == 0 else FULL for i in range(layers))
        tie = r.boolean("tie_word_embeddings", default=True)                # qwen/config.go:204
        if not tie:
            raise ConfigError(f"{where}: Gemma2 ties its output head to the embedding; "
                              "tie_word_embeddings=false is not supported")
        act = r.string("hidden_activation", default=r.raw.get("hidden_act") or "gelu_pytorch_tanh")
        if act not in ("gelu_pytorch_tanh", "gelu_tanh"):
            raise ConfigError(f"{where}: unsupported hidden_activation {act!r}")
        return cls(
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv,
            head_dim=head_dim,
            vocab_size=r.integer("vocab_size", minimum=1),
            intermediate_size=r.integer("intermediate_size", minimum=1),
            rope_theta=r.number("rope_theta", default=10000.0, minimum=0.0, exclusive=True),
            rms_norm_eps=r.number("rms_norm_eps", default=1e-6, minimum=0.0),
            query_pre_attn_scalar=r.number("query_pre_attn_scalar", default=float(head_dim),
                                           minimum=0.0, exclusive=True),
            attn_logit_softcapping=r.number("attn_logit_softcapping", default=0.0, minimum=0.0),
            final_logit_softcapping=r.number("final_logit_softcapping", default=0.0, minimum=0.0),
            sliding_window=window,
            max_position_embeddings=r.integer("max_position_embeddings", default=8192, minimum=1),
            layer_types=tuple(kinds),
            eos_token_id=r.int_or_list("eos_token_id"),
            tie_word_embeddings=tie,
            hidden_activation=act,
            model_type=r.string("model_type", default="gemma2"),
            architectures=r.string_list("architectures", default=("Gemma2ForCausalLM",)),
            torch_dtype=r.string("torch_dtype", default="bfloat16"),
        )

    def to_dict(self) -> dict:
        """The config.json that reads back to this object."""
        d = asdict(self)
        d["layer_types"] = list(self.layer_types)
        d["architectures"] = list(self.architectures)
        eos = list(self.eos_token_id)
        d["eos_token_id"] = eos[0] if len(eos) == 1 else eos
        if not eos:
            del d["eos_token_id"]
        return d
