"""The Qwen3 dense decoder put together from parts, by its configuration.

Per layer (src/engine/cpu_backend.zig:258-325): RMS norm, grouped-query attention with
per-head RMS norm of q and k before a rotate-half rotation, residual sum, RMS norm, SwiGLU
feed-forward, residual sum; then a final RMS norm and the output head, tied to the
embedding when the configuration says so.  Tensor names are Hugging Face's
(src/convert/hf.zig:95-129 lists them).  `layer_types` picks, layer by layer, the windowed
or the full attention mixer.
"""
from __future__ import annotations

from ..config import Qwen3Config, register_architecture
from ..parts import (GQAAttention, OutputHead, PreNormBlock, RMSNorm, RopeScaling, RotaryEmbedding, SwiGLUFeedForward,
                     TokenEmbedding)
from .spec import ModelSpec


def build_qwen3(cfg: Qwen3Config, max_positions: int = 0) -> ModelSpec:
    positions = max_positions or cfg.max_position_embeddings
    scaling = RopeScaling(**cfg.rope_scaling) if cfg.rope_scaling else None
    rope = RotaryEmbedding(cfg.rope_theta, cfg.rotary_dim, positions, pairing="half", scaling=scaling)
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = GQAAttention(cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                             p + "self_attn.", qk_norm_eps=cfg.rms_norm_eps, position=rope,
                             window=cfg.layer_window(i))
        ffn = SwiGLUFeedForward(cfg.hidden_size, cfg.intermediate_size, p + "mlp.")
        layers.append(PreNormBlock(
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm.weight"), mixer,
            RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm.weight"), ffn))
    embedding = TokenEmbedding(cfg.vocab_size, cfg.hidden_size, "model.embed_tokens.weight")
    head = OutputHead(cfg.hidden_size, cfg.vocab_size,
                      RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, "model.norm.weight"), "lm_head.weight",
                      tied_to="model.embed_tokens.weight" if cfg.tie_word_embeddings else None)
    return ModelSpec(cfg, embedding, layers, head)


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3, "qwen3")
