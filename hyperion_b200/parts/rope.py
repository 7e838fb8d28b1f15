"""Rotate-half rotary position encoding with a configurable base.

The table holds cos and sin of ``position * base**(-2i/d)`` for ``i < d/2``, computed in float64 and
kept in float32 (the reference computes the same angles in f64 and rounds the table to bfloat16:
helios/crates/helios-hal/src/reference.rs:71-87); the rotation is y[i] = x[i] c - x[i+d/2] s,
y[i+d/2] = x[i+d/2] c + x[i] s over the whole head (reference.rs:91-109).  Parameters: ``head_dim``,
``base``, ``max_positions``.  Tables are shared between parts with the same parameters.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import BuildContext, PositionEncoding, register_position
from .spec import PartSpec


def rotary_table(head_dim: int, base: float, max_positions: int) -> torch.Tensor:
    """[max_positions, head_dim/2, 2] float32: (cos, sin)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / head_dim)
    angle = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.stack([angle.cos(), angle.sin()], dim=-1).to(torch.float32).contiguous()


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.head_dim = int(spec.params["head_dim"])
        self.base = float(spec.params["base"])
        self.max_positions = int(spec.params.get("max_positions", build.max_positions))
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        key = ("rotary_table", self.head_dim, self.base, self.max_positions, str(build.device))
        if key not in build.shared:
            build.shared[key] = rotary_table(self.head_dim, self.base, self.max_positions).to(build.device)
        self.table = build.shared[key]

    def kernel_modules(self):
        return [("elementwise", {})]

    def apply_(self, x, heads, head_dim, positions):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        ops.rope_(x, heads, head_dim, positions, self.table)

    def apply_and_store_(self, x, q_heads, kv_heads, head_dim, positions, cache, token_row):
        if head_dim != self.head_dim:
            raise ValueError(f"rotary encoding built for head_dim {self.head_dim}, used with {head_dim}")
        ops.rope_kv_store_(x, q_heads, kv_heads, head_dim, positions, self.table, cache.kv, cache.block_table, token_row)


register_position("rope", RotaryEncoding)
