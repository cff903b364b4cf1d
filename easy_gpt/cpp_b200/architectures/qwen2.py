"""Qwen2 / Qwen2.5 dense decoder: typed configuration -> ModelSpec.

Tensor names are the reference's (src/models/layer_key_prefix.cpp:77-87,
src/models/embedding.cpp:30) plus ``lm_head.weight`` for an untied head, which
the reference never consumes (src/models/gpt_model.cpp:324-328).
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..registry import register_architecture


def build_spec(cfg: Qwen2Config) -> ModelSpec:
    layers = []
    for i in range(cfg.num_hidden_layers):
        prefix = f"model.layers.{i}"
        layers.append(LayerSpec(
            mixer=PartSpec("attention", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                qkv_bias=cfg.attention_bias, out_bias=cfg.attention_out_bias,
                window=cfg.layer_window(i)), prefix + ".self_attn"),
            feed_forward=PartSpec("swiglu", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                bias=cfg.mlp_bias), prefix + ".mlp"),
            mixer_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                prefix + ".input_layernorm"),
            feed_forward_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                                       prefix + ".post_attention_layernorm"),
            position=PartSpec("rope", dict(head_dim=cfg.head_dim, rotary_dim=cfg.head_dim,
                                           theta=cfg.rope_theta)),
        ))
    return ModelSpec(
        architecture="qwen2",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        layers=tuple(layers),
        run_order=tuple(RunEntry(layer=i, cache=i) for i in range(cfg.num_hidden_layers)),
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
                           "model.embed_tokens"),
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps), "model.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                         tied_to="model.embed_tokens" if cfg.tie_word_embeddings else None),
                         "lm_head"),
        bos_token_id=cfg.bos_token_id,
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("qwen2", Qwen2Config.from_dict, build_spec)
