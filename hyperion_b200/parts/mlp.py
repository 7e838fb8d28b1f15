"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

gate and up are fused into one [2I, H] matrix at load, gate rows first, as the reference places them
back to back for one matrix product (helios/crates/helios-hal/src/backends/hopper_sm90/backend.rs:95-106,
session.rs:779-793); silu(g) = g / (1 + exp(-g)) in float (kernels/elementwise.cu:28-37).
Parameters: ``hidden_size``, ``intermediate_size``.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from .base import BuildContext, FeedForward, WeightSpec, register_feed_forward
from .spec import PartSpec


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class SwiGLU(FeedForward):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])

    def weights(self) -> dict[str, WeightSpec]:
        return {"gate_proj.weight": WeightSpec((self.inter, self.hidden)), "up_proj.weight": WeightSpec((self.inter, self.hidden)),
                "down_proj.weight": WeightSpec((self.hidden, self.inter))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pair = [tensors["gate_proj.weight"], tensors["up_proj.weight"]]
        dtype = _common_dtype(pair)
        self.w_gate_up = torch.cat([t.to(dtype) for t in pair], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def kernel_modules(self):
        return [("elementwise", {}), ("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def forward(self, x, step):
        gate_up = ops.linear(x, self.w_gate_up, None, self.dtype)
        return ops.linear(ops.swiglu(gate_up), self.w_down, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_feed_forward("swiglu", SwiGLU)
