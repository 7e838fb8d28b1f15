from .basic import (add_rmsnorm, attention_generic, embedding, kv_store, place_tokens, raise_on_status, rope_, rope_kv_store_, sgemm_f32,
                    status_word, swiglu)
from .linear import gated_linear, linear
from .native import KernelError

__all__ = ["add_rmsnorm", "attention_generic", "embedding", "kv_store", "raise_on_status", "rope_", "rope_kv_store_", "sgemm_f32",
           "status_word", "swiglu", "linear", "gated_linear", "KernelError"]
