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


SMALL_PRODUCT_BYTES = 64 << 20  # weights of at most this many bytes go to the library at more than 32 rows

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
    """Which bfloat16 products go to the package's tcgen05 kernels.  ``auto``: every product of up to 64 rows with a
    reduction of at least 2,048 (the swapped kernel streams the weights as fast as or faster than the library at every
    decode batch, measured on a B200 at the 7B shapes: the output head over 152,064 tokens at 8 rows in 163 against 181 us,
    gate+up at 64 rows in 47 against 50 us, the whole step 4 % faster at batch 32; and it starts fetching weights while
    the kernel before it still runs), except products of a few tens of megabytes at more than 32 rows (qkv and o at the 7B
    shape: 12.6 and 11.2 us against the library's 9.1 and 8.3 at 64 rows; the step 4.54 against 4.61 ms at batch 64, 4.29
    against 4.33 at batch 48, even at batch 32, behind below).  Prompt-sized products stay with the library, whose kernels are up to 10 % ahead of
    this package's pair kernel, except gate+up with SwiGLU, which the pair kernel fuses (see ``gated_linear``)."""
    policy = gemm_policy()
    if policy == "library" or out_dtype not in (torch.bfloat16, torch.float32) or not gemm.supported(x, weight):
        return False
    if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
        return False
    if policy == "own":
        return True
    m, k = x.shape
    if m > 32 and weight.shape[0] * k * 2 <= SMALL_PRODUCT_BYTES:
        return False
    return k >= 2048 and m <= 64


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
        epilogue = gemm.EPI_F32 if out_dtype == torch.float32 else gemm.EPI_BF16
        if xin.shape[0] > gemm.PAIR_MIN_ROWS:  # only under HYPERION_B200_GEMM=own: prompt-sized products on pairs of SMs
            return gemm.gemm_pair_bf16(xin, weight, bias, epilogue)
        return gemm.gemm_bf16(xin, weight, bias, epilogue, leave_partials=may_leave_partials and out_dtype == torch.bfloat16)
    if not xin.is_contiguous():
        xin = xin.contiguous()
    if out_dtype == torch.bfloat16:
        b = bias if bias is None or bias.dtype == torch.bfloat16 else bias.to(torch.bfloat16)
        return torch.nn.functional.linear(xin, weight, b)
    y = torch.mm(xin, weight.t(), out_dtype=torch.float32)
    if bias is not None:
        y += bias.float()
    return y if out_dtype == torch.float32 else y.to(out_dtype)


def fuses_swiglu(m: int, k: int) -> bool:
    """Whether gate+up of ``m`` rows goes to the pair kernel with SwiGLU in its epilogue: from 512 rows on, when the rows
    fill their 256-row tiles to 85 % (measured at the 1.5B, 7B and 32B widths: 1.04 to 1.19 times the library's product
    followed by the SwiGLU kernel from 1,024 rows on, even at 512, behind below)."""
    policy = gemm_policy()
    if policy == "library":
        return False
    tiles = -(-m // 256)
    return m >= 512 and m >= 0.85 * tiles * 256


def gated_linear(x: torch.Tensor, weight: torch.Tensor, block: Optional[int], out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for a fused gate/up matrix ``weight`` [2I, H].  ``block`` None: the gate rows come first, then
    the up rows.  ``block`` = 128: rows alternate in runs of 128 gate rows and their 128 up rows
    (``ops.gemm.interleave_gate_up``), which lets a prompt-sized product apply SwiGLU in the epilogue of the pair kernel, so
    that the [tokens, 2I] projections never travel to memory and back."""
    from .basic import swiglu

    out_dtype = out_dtype or x.dtype
    if (block == gemm.SWIGLU_BLOCK and weight.dtype == torch.bfloat16 and out_dtype == torch.bfloat16 and x.dtype == torch.bfloat16
            and gemm.supported(x, weight) and fuses_swiglu(x.shape[0], x.shape[1])):
        return gemm.gemm_pair_bf16(x, weight, None, gemm.EPI_SWIGLU)
    return swiglu(linear(x, weight, None, out_dtype), block=block)
