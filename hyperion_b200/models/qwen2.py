"""Qwen2 dense (``Qwen2ForCausalLM``) expressed as parts.

Every layer is the pre-norm arrangement of grouped-query attention with q/k/v bias and rotate-half
RoPE, and a SwiGLU feed-forward, with RMSNorm before each; the head is ``lm_head.weight`` or the
embedding table when tied.  Tensor names are the Hugging Face names the reference expects
(ignition/src/hyperion_ignition/compiler/weights.py:177-207); a tied checkpoint that still carries
``lm_head.weight`` is tolerated (weights.py:233-236).
"""
from __future__ import annotations

from ..config.qwen2 import ARCHITECTURE, Qwen2Config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run
from .registry import Architecture, register_architecture


def build_spec(config: Qwen2Config) -> ModelSpec:
    position = PartSpec("rope", "", {"head_dim": config.head_dim, "base": config.rope_theta,
                                     "max_positions": config.max_position_embeddings})
    layers = []
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        norm = {"hidden_size": config.hidden_size, "eps": config.rms_norm_eps}
        layers.append(LayerSpec(
            arrangement="prenorm",
            mixer=PartSpec("gqa_attention", prefix + "self_attn.", {
                "hidden_size": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim, "bias": config.qkv_bias, "scale": config.attention_scale, "window": 0,
                "position": position}),
            feed_forward=PartSpec("swiglu", prefix + "mlp.", {"hidden_size": config.hidden_size,
                                                              "intermediate_size": config.intermediate_size}),
            norms={"input": PartSpec("rmsnorm", prefix + "input_layernorm.", norm),
                   "post_mixer": PartSpec("rmsnorm", prefix + "post_attention_layernorm.", norm)},
        ))
    sizes = {"vocab_size": config.vocab_size, "hidden_size": config.hidden_size}
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings,
        embedding=PartSpec("token_embedding", "model.embed_tokens.", sizes),
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rmsnorm", "model.norm.", {"hidden_size": config.hidden_size, "eps": config.rms_norm_eps}),
        head=PartSpec("linear_head", "lm_head.", {**sizes, "tied": config.tie_word_embeddings}),
        tolerated=("lm_head.weight",) if config.tie_word_embeddings else (),
    )


register_architecture(Architecture(ARCHITECTURE, Qwen2Config.from_hf_dict, build_spec, Qwen2Config.to_hf_dict))
