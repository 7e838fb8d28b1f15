"""Typed configuration of the Qwen2 dense decoder (``Qwen2ForCausalLM``).

Keys, defaults and refusals follow the reference's reader
(ignition/src/hyperion_ignition/compiler/model_config.py:96-169): ``num_key_value_heads`` defaults to
the number of heads (:133), ``head_dim`` to ``hidden_size / heads`` (:126-132), the RoPE base comes
from ``rope_theta`` or ``rope_parameters.rope_theta`` (:83-93), ``rms_norm_eps`` and
``tie_word_embeddings`` must be stated (:147-157), and RoPE scaling, sliding-window attention,
partial rotary embedding and any activation but SiLU are refused (:139-146).  A
``query_pre_attn_scalar`` that changes the attention scale is refused as the runtime does
(helios/crates/helios-hal/src/backends/hopper_sm90/forward.rs:81-84).  That Q, K and V carry a bias
is a property of the architecture, not of the file
(ignition/src/hyperion_ignition/compiler/architectures/qwen.py:20-21).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, ConfigReader

ARCHITECTURE = "Qwen2ForCausalLM"


@dataclass(frozen=True)
class Qwen2Config:
    num_hidden_layers: int
    hidden_size: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    eos_token_ids: tuple[int, ...] = ()
    qkv_bias: bool = True
    architecture: str = field(default=ARCHITECTURE)

    @property
    def attention_scale(self) -> float:
        return float(self.head_dim) ** -0.5

    @classmethod
    def from_hf_dict(cls, document: dict[str, Any]) -> "Qwen2Config":
        r = ConfigReader(document)
        found = r.raw("architectures")
        if not isinstance(found, list) or ARCHITECTURE not in found:
            raise ConfigError("architectures", f"must contain {ARCHITECTURE!r}, got {found!r}")
        heads = r.positive_int("num_attention_heads")
        hidden = r.positive_int("hidden_size")
        if r.has("head_dim"):
            head_dim = r.positive_int("head_dim")
        else:
            if hidden % heads:
                raise ConfigError("hidden_size", f"{hidden} is not divisible by num_attention_heads {heads}")
            head_dim = hidden // heads
        kv_heads = r.positive_int("num_key_value_heads") if r.has("num_key_value_heads") else heads
        if kv_heads > heads or heads % kv_heads:
            raise ConfigError("num_key_value_heads", f"{kv_heads} does not divide num_attention_heads {heads}")
        if head_dim % 2:
            raise ConfigError("head_dim", f"{head_dim} must be even (rotate-half position encoding)")
        if r.raw("rope_scaling"):
            raise ConfigError("rope_scaling", "is not supported")
        if r.raw("use_sliding_window"):
            raise ConfigError("use_sliding_window", "true is not supported")
        if r.raw("hidden_act") != "silu":
            raise ConfigError("hidden_act", f"{r.raw('hidden_act')!r} is not supported (only 'silu')")
        if r.raw("partial_rotary_factor", 1.0) != 1.0:
            raise ConfigError("partial_rotary_factor", "other than 1 is not supported")
        if r.has("query_pre_attn_scalar"):
            scale = r.positive_number("query_pre_attn_scalar") ** -0.5
            if abs(scale - head_dim ** -0.5) > 1e-12:
                raise ConfigError("query_pre_attn_scalar", "gives an attention scale other than head_dim**-0.5")
        return cls(
            num_hidden_layers=r.positive_int("num_hidden_layers"),
            hidden_size=hidden,
            intermediate_size=r.positive_int("intermediate_size"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=r.positive_int("vocab_size"),
            max_position_embeddings=r.positive_int("max_position_embeddings"),
            rope_theta=_rope_theta(r),
            rms_norm_eps=r.positive_number("rms_norm_eps"),
            tie_word_embeddings=r.boolean("tie_word_embeddings"),
            eos_token_ids=r.token_ids("eos_token_id"),
        )

    def to_hf_dict(self) -> dict[str, Any]:
        """The config.json document this configuration is read back from."""
        document: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "hidden_act": "silu",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "use_sliding_window": False,
        }
        if self.eos_token_ids:
            document["eos_token_id"] = list(self.eos_token_ids)
        return document


def _rope_theta(r: ConfigReader) -> float:
    if r.has("rope_theta"):
        return r.positive_number("rope_theta")
    parameters = r.raw("rope_parameters")
    if isinstance(parameters, dict):
        if parameters.get("rope_type", "default") != "default":
            raise ConfigError("rope_parameters.rope_type", f"{parameters.get('rope_type')!r} is not supported")
        if "rope_theta" in parameters:
            return r.positive_number("rope_parameters.rope_theta", parameters["rope_theta"])
    raise ConfigError("rope_theta", "is missing (neither at the top level nor in rope_parameters)")
