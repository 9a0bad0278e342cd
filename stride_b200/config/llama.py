"""Typed view of a Llama config.json.

The keys and defaults are those that arhaamatiq/stride reads (src/model.cpp:15-52):
hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, vocab_size
are required; num_key_value_heads defaults to the head count, head_dim to
hidden_size / heads, rms_norm_eps to 1e-5, rope_theta to 10000; rope_scaling may be
absent, "default" or "llama3" (factor 32, low_freq_factor 1, high_freq_factor 4,
original_max_position_embeddings 8192 by default); eos_token_id is an int or a list.
Unlike stride, any head ratio is accepted, max_position_embeddings sets the
capacity, and keys whose value this engine cannot honour (biases, another
activation) are refused instead of ignored.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


class ConfigError(ValueError):
    """A config.json key is missing or has a value this engine does not support."""


@dataclass(frozen=True)
class RopeScaling:
    rope_type: str = "default"           # "default" | "llama3"
    factor: float = 32.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: float = 8192.0


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling = field(default_factory=RopeScaling)
    max_position_embeddings: int = 2048
    tie_word_embeddings: Optional[bool] = None   # None: decided by the presence of lm_head.weight
    eos_token_ids: tuple = ()

    @staticmethod
    def from_dict(j: dict) -> "LlamaConfig":
        def need(key):
            if key not in j or j[key] is None:
                raise ConfigError(f"config.json: required key '{key}' is missing")
            v = j[key]
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                raise ConfigError(f"config.json: '{key}' must be a positive integer, got {v!r}")
            return v

        hidden = need("hidden_size")
        heads = need("num_attention_heads")
        kv_heads = j.get("num_key_value_heads") or heads
        head_dim = j.get("head_dim") or hidden // heads
        scaling = RopeScaling()
        r = j.get("rope_scaling")
        if r:
            kind = r.get("rope_type", r.get("type", "")) or "default"
            if kind == "llama3":
                scaling = RopeScaling(
                    "llama3", float(r.get("factor", 32.0)), float(r.get("low_freq_factor", 1.0)),
                    float(r.get("high_freq_factor", 4.0)), float(r.get("original_max_position_embeddings", 8192.0)))
                if scaling.high_freq_factor == scaling.low_freq_factor:
                    raise ConfigError("config.json: rope_scaling high_freq_factor equals low_freq_factor")
            elif kind != "default":
                raise ConfigError(f"config.json: unsupported rope type '{kind}' (supported: default, llama3)")
        for key in ("attention_bias", "mlp_bias"):
            if j.get(key):
                raise ConfigError(f"config.json: '{key}' = true is not supported (the decoder has no bias terms)")
        act = j.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act '{act}' is not supported (only 'silu')")
        eos = j.get("eos_token_id")
        eos_ids = () if eos is None else tuple(eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        cfg = LlamaConfig(
            hidden_size=hidden, intermediate_size=need("intermediate_size"), num_hidden_layers=need("num_hidden_layers"),
            num_attention_heads=heads, num_key_value_heads=int(kv_heads), head_dim=int(head_dim), vocab_size=need("vocab_size"),
            rms_norm_eps=float(j.get("rms_norm_eps", 1e-5)), rope_theta=float(j.get("rope_theta", 10000.0)),
            rope_scaling=scaling, max_position_embeddings=int(j.get("max_position_embeddings", 2048)),
            tie_word_embeddings=j.get("tie_word_embeddings"), eos_token_ids=eos_ids)
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.num_key_value_heads <= 0 or self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim <= 0 or self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even (rotary pairs)")
        if self.rms_norm_eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps {self.rms_norm_eps} must be positive")
        if self.max_position_embeddings <= 0:
            raise ConfigError("config.json: max_position_embeddings must be positive")

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to this configuration."""
        d = {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "head_dim": self.head_dim, "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings, "hidden_act": "silu",
        }
        if self.rope_scaling.rope_type != "default":
            s = self.rope_scaling
            d["rope_scaling"] = {"rope_type": s.rope_type, "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                                 "high_freq_factor": s.high_freq_factor,
                                 "original_max_position_embeddings": s.original_max_position_embeddings}
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
