"""LlamaForCausalLM as a `ModelSpec`: every layer is a pre-norm block of grouped-query
attention with rotary encoding and a SwiGLU feed-forward; tensor names are those of
arhaamatiq/stride's loader (src/model.cpp:204-232)."""
from __future__ import annotations

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .llama import LlamaConfig
from .registry import Architecture, register_architecture


def llama_model_spec(cfg: LlamaConfig) -> ModelSpec:
    s = cfg.rope_scaling
    position = PartSpec("rope", {
        "head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta,
        "scaling": {"rope_type": s.rope_type, "factor": s.factor, "low_freq_factor": s.low_freq_factor,
                    "high_freq_factor": s.high_freq_factor,
                    "original_max_position_embeddings": s.original_max_position_embeddings}})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("attention", {
                "hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "window": 0, "position": position},
                {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
                 "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight"}),
            feed_forward=PartSpec("swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
                                  {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
                                   "down": p + "mlp.down_proj.weight"}),
            mixer_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                {"weight": p + "input_layernorm.weight"}),
            feed_forward_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                       {"weight": p + "post_attention_layernorm.weight"}),
            block="prenorm"))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           {"weight": "model.embed_tokens.weight"}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, {"weight": "model.norm.weight"}),
        head=PartSpec("linear", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied": cfg.tie_word_embeddings},
                      {"weight": "lm_head.weight", "tied_to": "model.embed_tokens.weight"}),
        max_positions=cfg.max_position_embeddings, eos_token_ids=cfg.eos_token_ids)


register_architecture(Architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_model_spec), "llama")
