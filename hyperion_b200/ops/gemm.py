"""The package's own bfloat16 matrix product on tcgen05 tensor cores (``csrc/gemm_tcgen05.cu``).

``gemm_bf16(x, w)`` computes ``x w^T`` for ``x`` [M, K] and ``w`` [N, K].  Large M uses 128 x 256 tiles
with the activations on the 128-row side; M <= 64 swaps the operands so that the weight matrix
streams through the 128-row side once, with K split over several blocks when the weight matrix
alone has too few tiles to fill the GPU.  Epilogues: bfloat16 or float output with an optional bias,
and SwiGLU over a block-interleaved gate/up matrix (see ``interleave_gate_up``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .basic import status_word
from .native import KernelError, check, i32, library, ptr, require_cuda, sm_count, stream_ptr

EPI_BF16, EPI_F32, EPI_SWIGLU = 0, 1, 2
SWIGLU_BLOCK = 128  # the fused epilogue wants 128 gate rows followed by their 128 up rows, repeated
PAIR_MIN_ROWS = 128  # more rows than this: the pair kernel's 256-row tiles (when this package's kernels take a prompt-sized product at all)


def supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Operands this kernel takes: bfloat16, K-contiguous, 16-byte aligned rows (strides multiples of 8 elements)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.stride(1) == 1
            and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and x.shape[1] == w.shape[1])


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, H] gate and up matrices -> [2I, H] in blocks of 128 gate rows followed by the matching 128 up rows.
    I must be a multiple of 128."""
    inter, hidden = gate.shape
    if inter % SWIGLU_BLOCK:
        raise KernelError(f"the fused SwiGLU layout needs an intermediate size that is a multiple of {SWIGLU_BLOCK}, got {inter}")
    blocks = inter // SWIGLU_BLOCK
    return torch.stack([gate.view(blocks, SWIGLU_BLOCK, hidden), up.view(blocks, SWIGLU_BLOCK, hidden)], dim=1).reshape(2 * inter, hidden).contiguous()


def batch_tile_for(m: int) -> int:
    return 0 if m > 64 else (16 if m <= 16 else (32 if m <= 32 else 64))


def choose_splits(n: int, k: int, m: int = 64, sms: Optional[int] = None) -> int:
    """Split K so that the blocks fill the device (``sms`` multiprocessors, asked from the current device when absent):
    about two blocks per SM for up to 16 rows of activations (two blocks share an SM, one's start and epilogue pass under
    the other's stream, and the partial sums are small), about one per SM for more rows (the partial sums, ``splits`` times
    the output in float, cost more than the overlap gives); every split keeps at least 4 k-blocks."""
    sms = sms or sm_count()
    tiles = -(-n // 128)
    k_blocks = -(-k // 64)
    target = 2 * sms if m <= 16 else sms
    return max(1, min(target // tiles if tiles < target else 1, k_blocks // 4, 16))


@dataclass
class SplitSum:
    """A product whose split-K partial sums have not been added up yet: ``partials`` [splits, M, N] float32, to be
    summed in split order, plus ``bias``, rounded to ``dtype``.  A consumer that can read the pieces itself (the fused
    residual add + norm) saves the kernel that would add them; everyone else calls :meth:`tensor`."""

    partials: torch.Tensor
    bias: Optional[torch.Tensor]
    dtype: torch.dtype

    @property
    def shape(self) -> tuple[int, int]:
        return tuple(self.partials.shape[1:])

    def tensor(self) -> torch.Tensor:
        splits, m, n = self.partials.shape
        out = torch.empty((m, n), dtype=self.dtype, device=self.partials.device)
        bias_f = self.bias if self.bias is not None and self.bias.dtype == torch.float32 else None
        bias_h = self.bias if self.bias is not None and self.bias.dtype == torch.bfloat16 else None
        check(library("gemm_tcgen05").hb_splitk_reduce(ptr(self.partials), i32(splits), i32(m), i32(n), ptr(out), i32(out.stride(0)),
                                                       i32(self.dtype == torch.float32), ptr(bias_f), ptr(bias_h), stream_ptr()), "splitk_reduce")
        return out


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epilogue: int = EPI_BF16,
              out: Optional[torch.Tensor] = None, splits: Optional[int] = None, leave_partials: bool = False):
    """``leave_partials``: when K is split, return a :class:`SplitSum` instead of adding the pieces up."""
    require_cuda(x, w, bias)
    if not supported(x, w):
        raise KernelError("gemm_bf16: operands must be bfloat16, K-contiguous, with 16-byte aligned rows")
    m, k = x.shape
    n = w.shape[0]
    out_cols = n // 2 if epilogue == EPI_SWIGLU else n
    out_dtype = torch.float32 if epilogue == EPI_F32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, out_cols), dtype=out_dtype, device=x.device)
    if out.dtype != out_dtype or out.shape != (m, out_cols) or out.stride(1) != 1:
        raise KernelError("gemm_bf16: bad output tensor")
    bias_f = bias if bias is not None and bias.dtype == torch.float32 else None
    bias_h = bias if bias is not None and bias.dtype == torch.bfloat16 else None
    if bias is not None and bias_f is None and bias_h is None:
        raise KernelError("gemm_bf16: the bias is float32 or bfloat16")
    tile = batch_tile_for(m)
    if epilogue == EPI_SWIGLU:
        tile = 0  # the fused epilogue exists for the tile shape with activations on the 128-row side
    workspace = None
    if tile == 0:
        splits = 1
    else:
        splits = choose_splits(n, k, m) if splits is None else splits
        if splits > 1:
            workspace = torch.empty(splits * m * n, dtype=torch.float32, device=x.device)
    leave = int(leave_partials and workspace is not None and epilogue in (EPI_BF16, EPI_F32))
    lib = library("gemm_tcgen05")
    check(lib.hb_gemm_bf16(ptr(x), i32(x.stride(0)), ptr(w), i32(w.stride(0)), ptr(out), i32(out.stride(0)), ptr(bias_f), ptr(bias_h),
                           i32(m), i32(n), i32(k), i32(epilogue), i32(tile), i32(splits), ptr(workspace), i32(leave), ptr(status_word(x.device)),
                           stream_ptr()), "gemm_bf16")
    if leave:
        return SplitSum(workspace.view(splits, m, n), bias, out_dtype)
    return out


def gemm_pair_bf16(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epilogue: int = EPI_BF16,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x w^T`` on pairs of SMs (``csrc/gemm_pair_tcgen05.cu``: 256 x BN tiles, ``tcgen05.mma.cta_group::2``), for prompt-sized
    ``x``; the same operands and epilogues as :func:`gemm_bf16` in its tile shape."""
    require_cuda(x, w, bias)
    if not supported(x, w):
        raise KernelError("gemm_pair_bf16: operands must be bfloat16, K-contiguous, with 16-byte aligned rows")
    m, k = x.shape
    n = w.shape[0]
    out_cols = n // 2 if epilogue == EPI_SWIGLU else n
    out_dtype = torch.float32 if epilogue == EPI_F32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, out_cols), dtype=out_dtype, device=x.device)
    if out.dtype != out_dtype or out.shape != (m, out_cols) or out.stride(1) != 1:
        raise KernelError("gemm_pair_bf16: bad output tensor")
    bias_f = bias if bias is not None and bias.dtype == torch.float32 else None
    bias_h = bias if bias is not None and bias.dtype == torch.bfloat16 else None
    if bias is not None and bias_f is None and bias_h is None:
        raise KernelError("gemm_pair_bf16: the bias is float32 or bfloat16")
    check(library("gemm_pair_tcgen05").hb_gemm_pair_bf16(ptr(x), i32(x.stride(0)), ptr(w), i32(w.stride(0)), ptr(out), i32(out.stride(0)), ptr(bias_f),
                                                         ptr(bias_h), i32(m), i32(n), i32(k), i32(epilogue), ptr(status_word(x.device)), stream_ptr()),
          "gemm_pair_bf16")
    return out
