"""The Qwen3 dense decoder put together from parts.

Tensor names and what each layer holds follow the reference's binder
(crates/synaptix-models/llm/common/src/model.rs:723,742,770,783-788,845-857,861):
pre-norm blocks, grouped-query attention with per-head q/k RMSNorm before a
rotate-half rotation of the whole head, no projection bias, SwiGLU feed-forward,
final norm, output head tied to the embedding or separate.  Constants come from
``Qwen3Config`` (eps, theta, sizes, windows); scale is ``1/sqrt(head_dim)``
(crates/synaptix-models/llm/qwen3/src/config.rs:106).
"""
from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts import (Attention, Embedding, OutputHead, PreNormBlock, RMSNorm, RotaryHalf, SwiGLU)
from .decoder import DecoderModel


def build_qwen3(cfg: Qwen3Config) -> DecoderModel:
    embedding = Embedding("model.embed_tokens.weight", cfg.vocab_size, cfg.hidden_size)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = Attention(p + "self_attn.", cfg.hidden_size, cfg.num_attention_heads,
                          cfg.num_key_value_heads, cfg.head_dim,
                          position=RotaryHalf(cfg.head_dim, cfg.rope_theta),
                          qk_norm_eps=cfg.rms_norm_eps, window=cfg.layer_windows[i])
        layers.append(PreNormBlock(
            RMSNorm(p + "input_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            mixer,
            RMSNorm(p + "post_attention_layernorm.weight", cfg.hidden_size, cfg.rms_norm_eps),
            SwiGLU(p + "mlp.", cfg.hidden_size, cfg.intermediate_size)))
    final_norm = RMSNorm("model.norm.weight", cfg.hidden_size, cfg.rms_norm_eps)
    head = OutputHead("lm_head.weight", cfg.vocab_size, cfg.hidden_size, cfg.tie_word_embeddings, embedding)
    return DecoderModel(cfg, embedding, layers, final_norm, head, stop_token_ids=cfg.eos_token_ids)


register_architecture(Qwen3Config, build_qwen3)
