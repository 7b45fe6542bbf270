"""The dense Llama decoder laid out as a ModelSpec.

Arrangement and tensor names are those of the reference's model file
(model/llm/tiny_llama.cpp:29-34,53,61-62): per layer input_layernorm ->
self_attn (q/k/v/o_proj) -> residual -> post_attention_layernorm -> mlp
(gate/up/down_proj) -> residual; then model.norm and an untied lm_head.
"""
from __future__ import annotations

from ..config.model_config import LlamaConfig, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec


def build_llama_spec(cfg: LlamaConfig) -> ModelSpec:
    norm = lambda prefix: PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix)
    position = PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "max_position": cfg.max_position_embeddings})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        mixer = PartSpec("attention", {
            "hidden_size": cfg.hidden_size,
            "num_heads": cfg.num_attention_heads,
            "num_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "window": cfg.sliding_window,
            "position": position,
            "bias": cfg.attention_bias,
        }, p + ".self_attn")
        ffn = PartSpec("swiglu", {"hidden_size": cfg.hidden_size,
                                  "intermediate_size": cfg.intermediate_size, "bias": cfg.mlp_bias}, p + ".mlp")
        layers.append(LayerSpec("prenorm", {
            "norm1": norm(p + ".input_layernorm"),
            "mixer": mixer,
            "norm2": norm(p + ".post_attention_layernorm"),
            "ffn": ffn,
        }))
    head_params = {"hidden_size": cfg.hidden_size, "vocab_size": cfg.vocab_size}
    if cfg.tie_word_embeddings:
        head_params["tied_to"] = "model.embed_tokens.weight"
    spec = ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size},
                           "model.embed_tokens"),
        layers=tuple(layers),
        order=tuple(range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm"),
        head=PartSpec("lm_head", head_params, "lm_head"),
        eos_token_id=cfg.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture("LlamaForCausalLM", LlamaConfig, build_llama_spec)
