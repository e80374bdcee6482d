"""Qwen3 dense decoder as a plan of parts (src/paged/qwen3.rs:911-1037).

Every layer: pre-norm block, attention with q/k RMSNorm and full rotary
encoding, gated MLP.  The tensor names are the checkpoint's own
(src/paged/qwen3.rs:958-976, 919-928, 387-394, 324-326).  A layer's window
comes from `Qwen3Config.window_of_layer`, so layers may differ.
"""
from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = "model.layers.%d." % i
        layers.append(LayerSpec(
            mixer=PartSpec("paged_attention", p + "self_attn.", dict(
                hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, bias=cfg.attention_bias,
                qk_norm=True, eps=cfg.rms_norm_eps, window=cfg.window_of_layer(i),
                position=PartSpec("rotary", "", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta)))),
            feed_forward=PartSpec("gated_mlp", p + "mlp.", dict(
                hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                activation=cfg.hidden_act)),
            norms={"mixer": PartSpec("rms_norm", p + "input_layernorm.", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)),
                   "feed_forward": PartSpec("rms_norm", p + "post_attention_layernorm.",
                                            dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))},
            block="pre_norm"))
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
        embedding=PartSpec("token_embedding", "model.embed_tokens.",
                           dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size)),
        layers=layers,
        final_norm=PartSpec("rms_norm", "model.norm.", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)),
        head=PartSpec("linear_head", "lm_head.", dict(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                                                      tied=cfg.tie_word_embeddings)),
        order=list(range(cfg.num_hidden_layers)),
        max_positions=cfg.max_position_embeddings)


register_architecture(Qwen3Config.architecture, Qwen3Config.model_type, Qwen3Config, qwen3_plan)
