"""Qwen3 dense decoder (``Qwen3ForCausalLM``): configuration keys -> parts, order and tensor names.

Layer content follows miniserve/model/qwen3.py:326-346 (pre-norm block of attention and gated
MLP), attention options qwen3.py:56-106 (no biases, RMSNorm of q and k heads, half-split RoPE
with ``rope_theta``), tensor names miniserve/model/weight_map.py:19-46.
"""

from __future__ import annotations

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartSpec


def build_qwen3_spec(config: Qwen3Config) -> ModelSpec:
    position = PartSpec("rope", dict(head_dim=config.head_dim, theta=config.rope_theta))
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        layers.append(LayerSpec(
            prefix=prefix,
            mixer=PartSpec("attention", dict(
                hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
                num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim, qk_norm=True,
                eps=config.rms_norm_eps, position=position, window=None,
                q_name="self_attn.q_proj.weight", k_name="self_attn.k_proj.weight",
                v_name="self_attn.v_proj.weight", o_name="self_attn.o_proj.weight",
                q_norm_name="self_attn.q_norm.weight", k_norm_name="self_attn.k_norm.weight")),
            feed_forward=PartSpec("gated_mlp", dict(
                hidden_size=config.hidden_size, intermediate_size=config.intermediate_size,
                activation=config.hidden_act, gate_name="mlp.gate_proj.weight", up_name="mlp.up_proj.weight",
                down_name="mlp.down_proj.weight")),
            mixer_norm=PartSpec("rms", dict(name="input_layernorm.weight", size=config.hidden_size,
                                            eps=config.rms_norm_eps)),
            feed_forward_norm=PartSpec("rms", dict(name="post_attention_layernorm.weight", size=config.hidden_size,
                                                   eps=config.rms_norm_eps)),
        ))
    return ModelSpec(
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        embedding_name="model.embed_tokens.weight",
        layers=tuple(layers),
        order=tuple(LayerRun(index) for index in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms", dict(name="model.norm.weight", size=config.hidden_size, eps=config.rms_norm_eps)),
        output_name=None if config.tie_word_embeddings else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        # Qwen3 snapshots store lm_head.weight even when it is tied to the embedding.
        optional_names=("lm_head.weight",) if config.tie_word_embeddings else (),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_qwen3_spec)
