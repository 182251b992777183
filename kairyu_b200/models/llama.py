"""The Llama 3 / Qwen3 dense decoder as a spec (kairyu/models/llama.py:33-273).

Both architectures are one arrangement of the same parts; they differ in
whether q and k get a per-head RMSNorm (Qwen3, by architecture name as in
kairyu/models/config.py:190-200), and otherwise only in config values.
"""

from __future__ import annotations

from typing import Any, Mapping

from kairyu_b200.config.model_config import ModelConfig, parse_dense_config
from kairyu_b200.parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def dense_decoder_spec(config: ModelConfig, *, qk_norm: bool) -> ModelSpec:
    position = PartSpec(
        "rope",
        rotary_dim=config.head_dim,
        theta=config.rope_theta,
        scaling=config.rope_scaling,
        max_positions=config.max_position_embeddings,
    )
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}"
        layers.append(
            LayerSpec(
                prefix=prefix,
                block="pre_norm",
                mixer=PartSpec(
                    "gqa_attention",
                    prefix=f"{prefix}.self_attn",
                    hidden_size=config.hidden_size,
                    num_heads=config.num_attention_heads,
                    num_kv_heads=config.num_key_value_heads,
                    head_dim=config.head_dim,
                    qk_norm=qk_norm,
                    norm_eps=config.rms_norm_eps,
                    qkv_bias=config.attention_bias,
                    o_bias=config.attention_bias,
                    position=position,
                ),
                ffn=PartSpec(
                    "swiglu",
                    prefix=f"{prefix}.mlp",
                    hidden_size=config.hidden_size,
                    intermediate_size=config.intermediate_size,
                    activation=config.hidden_act,
                ),
                mixer_norm=PartSpec(
                    "rmsnorm", name=f"{prefix}.input_layernorm.weight", size=config.hidden_size, eps=config.rms_norm_eps
                ),
                ffn_norm=PartSpec(
                    "rmsnorm",
                    name=f"{prefix}.post_attention_layernorm.weight",
                    size=config.hidden_size,
                    eps=config.rms_norm_eps,
                ),
            )
        )
    return ModelSpec(
        embedding=PartSpec(
            "token_embedding",
            name="model.embed_tokens.weight",
            vocab_size=config.vocab_size,
            hidden_size=config.hidden_size,
        ),
        layers=tuple(layers),
        schedule=tuple(LayerCall(layer=i, cache_slot=i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", name="model.norm.weight", size=config.hidden_size, eps=config.rms_norm_eps),
        head=PartSpec(
            "linear_head",
            name="lm_head.weight",
            vocab_size=config.vocab_size,
            hidden_size=config.hidden_size,
            tied_to="model.embed_tokens.weight" if config.tie_word_embeddings else None,
        ),
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_position_embeddings=config.max_position_embeddings,
    )


def parse_llama(config: Mapping[str, Any]) -> ModelConfig:
    return parse_dense_config(config, "LlamaForCausalLM")


def parse_qwen3(config: Mapping[str, Any]) -> ModelConfig:
    return parse_dense_config(config, "Qwen3ForCausalLM")


def llama_spec(config: ModelConfig) -> ModelSpec:
    return dense_decoder_spec(config, qk_norm=False)


def qwen3_spec(config: ModelConfig) -> ModelSpec:
    return dense_decoder_spec(config, qk_norm=True)
