"""Dense projections y = x W^T (+ b) with W stored [out, in].

float32 weights go through the package's own FFMA kernel (the true 32-bit path: no tensor cores,
no reduced-precision matrix mode).  bfloat16 weights go either to the package's tcgen05 kernel
(``ops/gemm.py``; see ``_takes_own_kernel`` for which products) or to the library matrix product, as the
reference's engine does for every projection (``cublasGemmEx`` and ``cublasLtMatmul`` with a bias
epilogue: helios/crates/helios-hal/src/cuda/cublas.rs:158-188, cuda/cublaslt.rs:203-212,302);
accumulation is float, the bias is added before the one rounding to bfloat16, and the output head
keeps float logits (backends/hopper_sm90/session.rs:844-848).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import gemm
from .basic import sgemm_f32
from .native import KernelError, require_cuda


_policy: list = [None]


def gemm_policy() -> str:
    """``HYPERION_B200_GEMM`` (read once): ``auto`` (default), ``own`` (every bfloat16 product the tcgen05 kernel can take) or ``library``."""
    if _policy[0] is None:
        policy = os.environ.get("HYPERION_B200_GEMM", "auto")
        if policy not in ("auto", "own", "library"):
            raise KernelError(f"HYPERION_B200_GEMM must be auto, own or library, got {policy!r}")
        _policy[0] = policy
    return _policy[0]


def _takes_own_kernel(x: torch.Tensor, weight: torch.Tensor, bias, out_dtype) -> bool:
    """Which bfloat16 products go to the package's tcgen05 kernel.  ``auto``: with a reduction of at least 2,048, the
    products of up to 16 rows whose weight matrix has at most 65,536 rows (every projection; the output head over a
    large vocabulary is 0.3 % of a step faster in the library), and the products of up to 64 rows whose weight matrix
    has at most 4,096 rows (output and down projections).  There the swapped kernel streams the weights as fast as or faster than the library and starts
    fetching them while the kernel before it still runs (measured on a B200 at the 7B shapes: batch 8 decodes 3 %
    faster with every product here, batch 64 is fastest with the library's wide products).  Prompt-sized products stay
    with the library, whose 2-CTA kernels are ahead of this one-CTA kernel."""
    policy = gemm_policy()
    if policy == "library" or out_dtype not in (torch.bfloat16, torch.float32) or not gemm.supported(x, weight):
        return False
    if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
        return False
    if policy == "own":
        return True
    m, k = x.shape
    n = weight.shape[0]
    return k >= 2048 and ((m <= 16 and n <= 65536) or (m <= 64 and n <= 4096))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, may_leave_partials: bool = False):
    """``may_leave_partials``: the caller's result is only ever a residual delta, so a product that was split over K may
    come back as a :class:`hyperion_b200.ops.gemm.SplitSum` (the norm that adds the delta reads the pieces itself)."""
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
    if _takes_own_kernel(xin, weight, bias, out_dtype):
        return gemm.gemm_bf16(xin, weight, bias, gemm.EPI_F32 if out_dtype == torch.float32 else gemm.EPI_BF16,
                              leave_partials=may_leave_partials and out_dtype == torch.bfloat16)
    if not xin.is_contiguous():
        xin = xin.contiguous()
    if out_dtype == torch.bfloat16:
        b = bias if bias is None or bias.dtype == torch.bfloat16 else bias.to(torch.bfloat16)
        return torch.nn.functional.linear(xin, weight, b)
    y = torch.mm(xin, weight.t(), out_dtype=torch.float32)
    if bias is not None:
        y += bias.float()
    return y if out_dtype == torch.float32 else y.to(out_dtype)
