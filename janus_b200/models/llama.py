"""The Llama dense decoder as data: a `ModelSpec` made from a `LlamaConfig`.

Checkpoint names are the ones the reference looks up first
(crates/janus-engine/examples/inference.rs:33-77,285-291); the layer is the
reference's block (crates/janus-engine/src/model/block.rs:190-458): RMSNorm,
grouped-query attention with rotary positions, RMSNorm, SwiGLU, pre-norm
residuals.  Every size and constant comes from the configuration.
"""
from __future__ import annotations

from typing import List

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_spec(config: LlamaConfig) -> ModelSpec:
    position = PartSpec("rotary", dict(
        head_dim=config.head_dim, theta=config.rope_theta, max_positions=config.max_position_embeddings,
        scaling=None if config.rope_scaling is None else config.rope_scaling.to_dict()))
    layers: List[LayerSpec] = []
    for i in range(config.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            mixer=PartSpec("gqa_attention", dict(
                hidden_size=config.hidden_size, num_heads=config.num_attention_heads,
                num_kv_heads=config.num_key_value_heads, head_dim=config.head_dim, position=position, window=0),
                weights=dict(q=p + "self_attn.q_proj.weight", k=p + "self_attn.k_proj.weight",
                             v=p + "self_attn.v_proj.weight", o=p + "self_attn.o_proj.weight")),
            feed_forward=PartSpec("swiglu", dict(
                hidden_size=config.hidden_size, intermediate_size=config.intermediate_size),
                weights=dict(gate=p + "mlp.gate_proj.weight", up=p + "mlp.up_proj.weight",
                             down=p + "mlp.down_proj.weight")),
            mixer_norm=PartSpec("rms_norm", dict(width=config.hidden_size, eps=config.rms_norm_eps),
                                weights=dict(gamma=p + "input_layernorm.weight")),
            feed_forward_norm=PartSpec("rms_norm", dict(width=config.hidden_size, eps=config.rms_norm_eps),
                                       weights=dict(gamma=p + "post_attention_layernorm.weight")),
            arrangement="pre_norm"))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", dict(width=config.hidden_size, eps=config.rms_norm_eps),
                            weights=dict(gamma="model.norm.weight")),
        embedding_weight="model.embed_tokens.weight",
        head_weight=None if config.tie_word_embeddings else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        # a tied checkpoint may still store the head; rotary tables of older exports are not weights
        ignorable_weights=("lm_head.weight",) if config.tie_word_embeddings else (),
    )


def build_llama(config: LlamaConfig, dtype, device):
    from ..engine.model import DecoderModel
    return DecoderModel(llama_spec(config), dtype, device)


def llama_weight_specs(config: LlamaConfig):
    from ..engine.model import model_weight_specs
    return model_weight_specs(llama_spec(config))


register_architecture(LlamaConfig.ARCHITECTURE, LlamaConfig, build_llama, llama_weight_specs)
