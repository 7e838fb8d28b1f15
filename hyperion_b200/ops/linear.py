"""Dense projections y = x W^T (+ b) with W stored [out, in].

float32 weights go through the package's own FFMA kernel (the true 32-bit path: no tensor cores,
no reduced-precision matrix mode).  bfloat16 weights go through the library matrix product, as the
reference's engine does for every projection (``cublasGemmEx`` and ``cublasLtMatmul`` with a bias
epilogue: helios/crates/helios-hal/src/cuda/cublas.rs:158-188, cuda/cublaslt.rs:203-212,302);
accumulation is float, the bias is added before the one rounding to bfloat16, and the output head
keeps float logits (backends/hopper_sm90/session.rs:844-848).
"""
from __future__ import annotations

from typing import Optional

import torch

from .basic import sgemm_f32
from .native import KernelError, require_cuda


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    require_cuda(x, weight, bias)
    out_dtype = out_dtype or x.dtype
    if weight.dtype == torch.float32:
        xin = x if x.dtype == torch.float32 else x.float()
        b = bias if bias is None or bias.dtype == torch.float32 else bias.float()
        y = sgemm_f32(xin, weight, b)
        return y if out_dtype == torch.float32 else y.to(out_dtype)
    if weight.dtype != torch.bfloat16:
        raise KernelError(f"linear: weights are float32 or bfloat16, got {weight.dtype}")
    xin = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if not xin.is_contiguous():
        xin = xin.contiguous()
    if out_dtype == torch.bfloat16:
        b = bias if bias is None or bias.dtype == torch.bfloat16 else bias.to(torch.bfloat16)
        return torch.nn.functional.linear(xin, weight, b)
    y = torch.mm(xin, weight.t(), out_dtype=torch.float32)
    if bias is not None:
        y += bias.float()
    return y if out_dtype == torch.float32 else y.to(out_dtype)
