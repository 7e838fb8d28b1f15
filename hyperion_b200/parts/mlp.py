"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases.

gate and up are fused into one [2I, H] matrix at load, as the reference places them back to back for one
matrix product (helios/crates/helios-hal/src/backends/hopper_sm90/backend.rs:95-106, session.rs:779-793);
silu(g) = g / (1 + exp(-g)) in float (kernels/elementwise.cu:28-37).  In bfloat16, when the intermediate size
allows it, the rows alternate in runs of 128 gate rows and their 128 up rows, so that a prompt-sized
product can apply SwiGLU in its epilogue (``ops.gated_linear``); otherwise the gate rows come first.
Parameters: ``hidden_size``, ``intermediate_size``.
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import gemm
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
        if dtype == torch.bfloat16 and self.inter % gemm.SWIGLU_BLOCK == 0:
            self.block = gemm.SWIGLU_BLOCK
            self.w_gate_up = gemm.interleave_gate_up(pair[0], pair[1])
        else:
            self.block = None
            self.w_gate_up = torch.cat([t.to(dtype) for t in pair], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"].contiguous()

    def kernel_modules(self):
        if self.dtype == torch.float32:
            return [("elementwise", {}), ("sgemm_f32", {})]
        return [("elementwise", {}), ("gemm_tcgen05", {}), ("gemm_pair_tcgen05", {})]

    def forward(self, x, step):
        act = ops.gated_linear(x, self.w_gate_up, self.block, self.dtype)
        return ops.linear(act, self.w_down, None, self.dtype, may_leave_partials=True)  # the result is a residual delta


register_feed_forward("swiglu", SwiGLU)
