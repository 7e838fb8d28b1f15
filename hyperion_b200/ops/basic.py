"""The row-wise operations and the 32-bit matrix product, as functions over torch tensors."""
from __future__ import annotations

import torch

from .native import KernelError, check, f32, i32, is_bf16, library, ptr, require_cuda, stream_ptr

_STATUS: dict[int, torch.Tensor] = {}
STATUS_BITS = {1: "a block-table entry that had to be valid was missing", 2: "a token id outside the vocabulary",
               4: "a position beyond the position table", 8: "a bounded wait inside a kernel ran out",
               0x100: "(in the tile-shaped GEMM)", 0x200: "(in the swapped GEMM)", 0x400: "(in the TMA attention, tile shape)",
               0x800: "(in the TMA attention, token shape)", 0x1000: "(in the tcgen05 attention)"}


def status_word(device: torch.device) -> torch.Tensor:
    """The int32 word kernels set bits in instead of faulting; one per device."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _STATUS:
        _STATUS[index] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
    return _STATUS[index]


def raise_on_status(device: torch.device) -> None:
    """Read the status word (this waits for the device) and raise if a kernel reported a problem."""
    word = status_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        reasons = [text for bit, text in STATUS_BITS.items() if value & bit]
        raise KernelError(f"a kernel reported (status word {value:#x}): " + "; ".join(reasons))


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = float(table[ids[t]]); ids int32 on the device."""
    require_cuda(table, ids)
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    lib = library("elementwise")
    check(lib.hb_embedding(ptr(table), i32(is_bf16(table)), ptr(ids), ptr(out), i32(tokens), i32(hidden), i32(vocab),
                           ptr(status_word(table.device)), stream_ptr()), "embedding")
    return out


def place_tokens(ids: torch.Tensor, source: torch.Tensor, pairs: torch.Tensor) -> None:
    """ids[pairs[i, 0]] = source[pairs[i, 1]] on the device (all int32); the caller has checked the pairs."""
    require_cuda(ids, source, pairs)
    check(library("elementwise").hb_place_tokens(ptr(ids), ptr(source), ptr(pairs), i32(pairs.numel() // 2), stream_ptr()), "place_tokens")


def add_rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
                rows: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of ``h (+ delta)`` times ``weight``.

    Without ``rows`` the sum is written back into ``h`` (float residual stream) and every row is
    normalised; with ``rows`` (int32 indices) only those rows are read and ``h`` is left alone.
    ``delta`` is a tensor, None, or a ``SplitSum`` (a product whose split-K pieces this kernel adds up itself).
    """
    from .gemm import SplitSum

    pieces = delta if isinstance(delta, SplitSum) else None
    hidden = h.shape[-1]
    if pieces is not None:
        fits = (out_dtype == torch.bfloat16 and pieces.dtype == torch.bfloat16 and hidden % 8 == 0 and hidden <= 16384
                and pieces.shape == tuple(h.shape) and pieces.partials.is_contiguous())
        delta = None if fits else pieces.tensor()
        pieces = pieces if fits else None
    require_cuda(h, delta, weight, rows)
    if h.dtype != torch.float32 or weight.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("add_rmsnorm: the residual stream and the norm weight are float32")
    n_rows = rows.numel() if rows is not None else h.shape[0]
    if out is None:
        out = torch.empty((n_rows, hidden), dtype=out_dtype, device=h.device)
    if delta is not None and (delta.shape != h.shape or not delta.is_contiguous()):
        raise KernelError("add_rmsnorm: delta must have the shape of h")
    lib = library("elementwise")
    write_h = i32(0 if rows is not None else 1)
    if pieces is not None:
        bias = pieces.bias
        bias_f = bias if bias is not None and bias.dtype == torch.float32 else None
        bias_h = bias if bias is not None and bias.dtype == torch.bfloat16 else None
        check(lib.hb_add_rmsnorm_splits(ptr(h), ptr(pieces.partials), i32(pieces.partials.shape[0]), i32(h.shape[0]), ptr(bias_f), ptr(bias_h),
                                        ptr(weight), ptr(out), ptr(rows), i32(n_rows), i32(hidden), f32(eps), write_h, stream_ptr()), "add_rmsnorm")
        return out
    check(lib.hb_add_rmsnorm(ptr(h), ptr(delta), i32(is_bf16(delta) if delta is not None else 0), ptr(weight), ptr(out),
                             i32(is_bf16(out)), ptr(rows), i32(n_rows), i32(hidden), f32(eps), write_h,
                             stream_ptr()), "add_rmsnorm")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, block: int | None = None) -> torch.Tensor:
    """[tokens, 2I] -> silu(gate) * up, [tokens, I].  ``block``: gate and up columns alternate in runs of that many columns
    (``block`` gate columns, then their up columns); None: all gate columns first."""
    require_cuda(gate_up)
    tokens, twice = gate_up.shape
    inter = twice // 2
    block = inter if block is None else block
    if block <= 0 or inter % block:
        raise KernelError(f"swiglu: runs of {block} columns do not divide {inter}")
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    lib = library("elementwise")
    for start in range(0, tokens, 65535):
        count = min(65535, tokens - start)
        check(lib.hb_swiglu(ptr(gate_up[start:]), ptr(out[start:]), i32(is_bf16(gate_up)), i32(count), i32(inter), i32(block), stream_ptr()), "swiglu")
    return out


def rope_(x: torch.Tensor, heads: int, head_dim: int, positions: torch.Tensor, table: torch.Tensor) -> None:
    """Rotate the first ``heads`` heads of every row of ``x`` in place; table [max_pos, head_dim/2, 2] float."""
    require_cuda(x, positions, table)
    if x.stride(-1) != 1 or table.dtype != torch.float32 or table.shape[1] * 2 != head_dim:
        raise KernelError("rope: bad layout")
    lib = library("elementwise")
    check(lib.hb_rope(ptr(x), i32(is_bf16(x)), ptr(positions), ptr(table), i32(x.shape[0]), i32(x.stride(0)), i32(heads),
                      i32(head_dim), i32(table.shape[0]), ptr(status_word(x.device)), stream_ptr()), "rope")


def kv_store(src: torch.Tensor, k_offset: int, v_offset: int, cache: torch.Tensor, block_table: torch.Tensor,
             token_row: torch.Tensor, positions: torch.Tensor) -> None:
    """Write each token's keys and values (columns of ``src``) into ``cache`` [pages, 2, kv_heads, page, d]."""
    require_cuda(src, cache, block_table, token_row, positions)
    pages, two, kv_heads, page_size, head_dim = cache.shape
    if src.dtype != cache.dtype or two != 2 or not cache.is_contiguous() or src.stride(-1) != 1:
        raise KernelError("kv_store: source and cache must share their element type and be dense")
    lib = library("elementwise")
    check(lib.hb_kv_store(ptr(src), i32(is_bf16(src)), i32(src.shape[0]), i32(src.stride(0)), i32(k_offset), i32(v_offset),
                          ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row), ptr(positions), i32(kv_heads),
                          i32(head_dim), i32(page_size), i32(pages), ptr(status_word(src.device)), stream_ptr()), "kv_store")


def rope_kv_store_(x: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, positions: torch.Tensor, table: torch.Tensor,
                   cache: torch.Tensor, block_table: torch.Tensor, token_row: torch.Tensor) -> None:
    """RoPE on the q heads of ``x`` = [q | k | v] in place, rotated keys and the values written to ``cache``."""
    require_cuda(x, positions, table, cache, block_table, token_row)
    pages, two, cache_heads, page_size, cache_dim = cache.shape
    if (x.dtype != cache.dtype or x.stride(-1) != 1 or table.dtype != torch.float32 or table.shape[1] * 2 != head_dim
            or cache_heads != kv_heads or cache_dim != head_dim or not cache.is_contiguous()):
        raise KernelError("rope_kv_store: bad layout")
    lib = library("elementwise")
    check(lib.hb_rope_kv_store(ptr(x), i32(is_bf16(x)), i32(x.shape[0]), i32(x.stride(0)), i32(q_heads), i32(kv_heads), i32(head_dim),
                               ptr(positions), ptr(table), i32(table.shape[0]), ptr(cache), ptr(block_table), i32(block_table.shape[1]),
                               ptr(token_row), i32(page_size), i32(pages), ptr(status_word(x.device)), stream_ptr()), "rope_kv_store")


def attention_generic(q: torch.Tensor, heads: int, cache: torch.Tensor, block_table: torch.Tensor, token_row: torch.Tensor,
                      positions: torch.Tensor, scale: float, window: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of every token over its request's pages; q is [tokens, >= heads*d] (a view is fine)."""
    require_cuda(q, cache, block_table, token_row, positions)
    pages, two, kv_heads, page_size, head_dim = cache.shape
    tokens = q.shape[0]
    if out is None:
        out = torch.empty((tokens, heads * head_dim), dtype=q.dtype, device=q.device)
    if q.dtype != cache.dtype or q.stride(-1) != 1:
        raise KernelError("attention: queries and cache must share their element type")
    lib = library("attention_generic")
    check(lib.hb_attention_generic(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), i32(is_bf16(q)), ptr(cache),
                                   ptr(block_table), i32(block_table.shape[1]), ptr(token_row), ptr(positions), i32(tokens),
                                   i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale), i32(window or 0),
                                   ptr(status_word(q.device)), stream_ptr()), "attention_generic")
    return out


def sgemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] (rows may be strided) times weight [N, K] transposed, plus bias, in plain float."""
    require_cuda(x, weight, bias)
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.stride(-1) != 1 or not weight.is_contiguous():
        raise KernelError("sgemm_f32: float32 operands with unit inner stride")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError(f"sgemm_f32: x has {k} columns, weight {weight.shape[1]}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    lib = library("sgemm_f32")
    step = 65535 * 64
    for start in range(0, m, step):
        count = min(step, m - start)
        check(lib.hb_sgemm_f32(ptr(x[start:]), ptr(weight), ptr(bias), ptr(out[start:]), i32(count), i32(n), i32(k),
                               i32(x.stride(0)), i32(out.stride(0)), stream_ptr()), "sgemm_f32")
    return out
