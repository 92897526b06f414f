"""Qwen2-MoE: from the typed config to a ``ModelSpec``.

This is the only file that knows how this architecture chooses its parts:
attention on every layer with Q/K/V biases and full-head NeoX rotation
(``config.h:25`` calls it "bit-for-bit the Qwen2 path"), softmax scale
``1/sqrt(head_dim)`` (src/model/qwen2.cc:890), a sliding window on layers at or
beyond ``max_window_layers`` when ``use_sliding_window`` is set, a routed
feed-forward on layers where ``(i+1) % decoder_sparse_step == 0`` and ``i`` is not
in ``mlp_only_layers`` and a dense SwiGLU elsewhere, a sigmoid-gated shared
expert, routed scale 1, and an optionally tied head.
"""
from __future__ import annotations

import math

from ..config.model_config import Qwen2MoeConfig
from ..parts.specs import (AttentionSpec, LayerSpec, ModelSpec, MoeSpec, RmsNormSpec, RopeSpec,
                           RunEntry, SwiGluSpec)


def build_spec(cfg: Qwen2MoeConfig) -> ModelSpec:
    norm = RmsNormSpec(size=cfg.hidden_size, eps=cfg.rms_norm_eps)
    rope = RopeSpec(head_dim=cfg.head_dim, rotary_dim=cfg.head_dim, theta=cfg.rope_theta)
    layers = []
    for i in range(cfg.num_hidden_layers):
        mixer = AttentionSpec(
            hidden=cfg.hidden_size, heads=cfg.num_attention_heads,
            kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
            qkv_bias=cfg.attention_bias, scale=1.0 / math.sqrt(cfg.head_dim),
            window=cfg.layer_window(i), position=rope)
        if cfg.layer_is_sparse(i):
            ffn = MoeSpec(
                hidden=cfg.hidden_size, num_experts=cfg.num_experts,
                top_k=cfg.num_experts_per_tok, expert_intermediate=cfg.moe_intermediate_size,
                renormalize=cfg.norm_topk_prob, routed_scale=1.0,
                shared=(SwiGluSpec(hidden=cfg.hidden_size,
                                   intermediate=cfg.shared_expert_intermediate_size)
                        if cfg.shared_expert_intermediate_size > 0 else None),
                shared_gated=True)
        else:
            ffn = SwiGluSpec(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size)
        layers.append(LayerSpec(prefix=f"model.layers.{i}", input_norm=norm, mixer=mixer,
                                post_norm=norm, ffn=ffn))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab_size, hidden=cfg.hidden_size,
        layers=tuple(layers), schedule=tuple(RunEntry(i) for i in range(len(layers))),
        final_norm=norm, tied_head=cfg.tie_word_embeddings)
