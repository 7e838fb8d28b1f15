"""RMSNorm with the residual add fused in.

y = x * rsqrt(mean(x^2) + eps) * weight, the weight multiplying after the normalisation
(helios/crates/helios-hal/kernels/rmsnorm.cu:22-58); the fused form first adds the pending delta into
the residual stream (rmsnorm.cu:66-122).  The stream, the sum of squares and the products are float;
the result is rounded once to the activation type.  Parameters: ``hidden_size``, ``eps``.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from .. import ops
from .base import BuildContext, Norm, WeightSpec, register_norm
from .spec import PartSpec


class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.hidden = int(spec.params["hidden_size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weights(self) -> dict[str, WeightSpec]:
        return {"weight": WeightSpec((self.hidden,), init="one_plus_normal")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].to(torch.float32).contiguous()

    def kernel_modules(self):
        return [("elementwise", {})]

    def forward(self, h, delta, rows=None):
        return ops.add_rmsnorm(h, delta, self.weight, self.eps, self.dtype, rows)


register_norm("rmsnorm", RMSNorm)
