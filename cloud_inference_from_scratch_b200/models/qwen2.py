"""Qwen2 dense decoder: from its typed configuration to a model description.

The arrangement is the reference's ``Qwen2CausalLM`` (src/cloud_engine/model.py:163-228):
token embedding; per layer RMSNorm -> grouped-query attention with q/k/v biases and
NeoX rotary -> residual -> RMSNorm -> SwiGLU -> residual; final RMSNorm; LM head tied to
the embedding or a matrix of its own.  Tensor names are those of the weight files
(src/cloud_engine/weights.py:36-78).
"""

from __future__ import annotations

from ..config.model_config import Qwen2Config
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def qwen2_spec(config: Qwen2Config) -> ModelSpec:
    position = PartSpec(
        "rope_neox",
        dict(
            head_dim=config.head_dim,
            rotary_dim=config.head_dim,
            theta=config.rope_theta,
            max_positions=config.max_position_embeddings,
        ),
    )
    layers = []
    for index in range(config.num_hidden_layers):
        norm_params = dict(hidden_size=config.hidden_size, eps=config.rms_norm_eps)
        layers.append(
            LayerSpec(
                prefix=f"model.layers.{index}.",
                block=PartSpec("prenorm_residual"),
                mixer=PartSpec(
                    "attention",
                    dict(
                        hidden_size=config.hidden_size,
                        num_heads=config.num_attention_heads,
                        num_kv_heads=config.num_key_value_heads,
                        head_dim=config.head_dim,
                        qkv_bias=config.attention_bias,
                        window=0,
                        position=position,
                    ),
                    prefix="self_attn.",
                ),
                feed_forward=PartSpec(
                    "swiglu",
                    dict(hidden_size=config.hidden_size, intermediate_size=config.intermediate_size),
                    prefix="mlp.",
                ),
                mixer_norm=PartSpec("rmsnorm", norm_params, prefix="input_layernorm."),
                feed_forward_norm=PartSpec(
                    "rmsnorm", norm_params, prefix="post_attention_layernorm."
                ),
            )
        )
    tied = config.tie_word_embeddings
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        embedding_tensor="model.embed_tokens.weight",
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec(
            "rmsnorm", dict(hidden_size=config.hidden_size, eps=config.rms_norm_eps)
        ),
        final_norm_prefix="model.norm.",
        head_tensor="model.embed_tokens.weight" if tied else "lm_head.weight",
        max_positions=config.max_position_embeddings,
        eos_token_id=config.eos_token_id,
        # a tied model may still ship the head; it is accepted and not read (weights.py:31-33,103)
        optional_tensors=("lm_head.weight",) if tied else (),
    )


register_architecture("Qwen2ForCausalLM", "qwen2", Qwen2Config.from_dict, qwen2_spec, replace=True)
