"""Qwen3 dense as data: a ``ModelSpec`` made of registered parts.

Layer structure, tensor names and order of operations follow the reference's
only model (src/model/qwen_model.cu:55-95 for names, :97-191 for the forward):
pre-norm blocks of grouped-query attention (per-head RMSNorm on q and k before
the rotation, rotate-half rotary encoding over the full head) and a SwiGLU
feed-forward, a final RMSNorm and an output head that may share the embedding
matrix.
"""
from __future__ import annotations

from ..config.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.qwen3 import Qwen3Config
from .registry import register_architecture


def qwen3_spec(cfg: Qwen3Config) -> ModelSpec:
    rope = PartSpec("rotary", dict(head_dim=cfg.head_dim, rotary_dim=cfg.head_dim,
                                   theta=cfg.rope_theta, max_positions=cfg.max_position_embeddings))
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        norm = dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)
        layers.append(LayerSpec(
            arrangement="pre_norm",
            mixer=PartSpec("gqa_attention", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim,
                qk_norm=True, qk_norm_eps=cfg.rms_norm_eps, window=None,
                scale=None), prefix=f"{p}.self_attn"),
            feed_forward=PartSpec("swiglu_mlp", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size),
                prefix=f"{p}.mlp"),
            norms=(PartSpec("rms_norm", norm, prefix=f"{p}.input_layernorm"),
                   PartSpec("rms_norm", norm, prefix=f"{p}.post_attention_layernorm")),
            position=rope,
        ))
    return ModelSpec(
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size,
                                                   hidden_size=cfg.hidden_size),
                           prefix="model.embed_tokens"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps),
                            prefix="model.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                      tied_to="model.embed_tokens.weight"
                                      if cfg.tie_word_embeddings else None),
                      prefix="lm_head"),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_spec)
