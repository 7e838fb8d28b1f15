"""Tensor-core attention over the paged bfloat16 cache: planning on the host and the two launches.

A step's rows are divided by length: rows of more than ``TOKEN_SHAPE_MAX`` tokens are cut into tiles
of ``tile_tokens`` tokens (times the heads of one key/value group = the virtual rows of a block: up to
256 for the tcgen05 kernel, 64 for the others); the tokens of shorter rows (decoded tokens, very short
portions) each get blocks of their own, with the keys split over several blocks when the batch alone
would not fill the GPU.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import host as host_runtime
from .basic import status_word
from .native import KernelError, check, f32, i32, library, ptr, require_cuda, sm_count, stream_ptr

TOKEN_SHAPE_MAX = 4  # at most csrc/attention_tma.cu's FRESH_TOKENS: its producer fetches older keys before the kernel ahead has finished
TILE_ROWS = 64
TC_TILE_ROWS = 256  # csrc/attention_tcgen05.cu: two halves of 128 rows per block
KEY_TILE = 64
BLOCKS_PER_SM = 2  # two blocks of the token shape fit one SM


def supported(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def uses_tma(head_dim: int, page_size: int) -> bool:
    """Head sizes that are multiples of 64 with pages of 8 to 64 tokens take the TMA-fed kernels."""
    return head_dim % 64 == 0 and 8 <= page_size <= 64


def _entry(head_dim: int, page_size: int, shape: str):
    if uses_tma(head_dim, page_size):
        return getattr(library("attention_tma", HB_HEAD_DIM=head_dim), f"hb_attention_tma_{shape}")
    return getattr(library("attention_bf16", HB_HEAD_DIM=head_dim), f"hb_attention_{shape}")


def uses_tcgen05(head_dim: int, page_size: int) -> bool:
    """Head sizes 64 and 128 with pages of 8 to 64 tokens: prompt portions take the tcgen05 kernel (256-row tiles)."""
    return head_dim in (64, 128) and 8 <= page_size <= 64


def tile_rows(head_dim: int, page_size) -> int:
    """Virtual rows (tokens x heads of a group) per tile of the kernel that will run."""
    return TC_TILE_ROWS if page_size is not None and uses_tcgen05(head_dim, page_size) else TILE_ROWS


def tile_tokens(heads: int, kv_heads: int, rows: int = TILE_ROWS) -> int:
    return rows // min(heads // kv_heads, rows)


def plan(rows, tokens_per_tile: int) -> tuple[np.ndarray, np.ndarray]:
    """(tiles as flat triples [first token, count, batch row], items = flat token indices), int32 arrays, made by the
    host runtime from the rows' token counts (rows follow one another in the flat batch)."""
    counts = host_runtime.ints(rows.counts if hasattr(rows, "counts") else [row.count for row in rows])
    tiles = np.empty(3 * int((-(-counts // tokens_per_tile)).sum()), dtype=np.int32)
    items = np.empty(int(counts.sum()), dtype=np.int32)
    n_tiles, n_items = ctypes.c_int(), ctypes.c_int()
    host_runtime.check(host_runtime.library().hb_plan_attention(len(counts), host_runtime.address(counts), tokens_per_tile, TOKEN_SHAPE_MAX,
                                                                host_runtime.address(tiles), ctypes.byref(n_tiles), host_runtime.address(items),
                                                                ctypes.byref(n_items)))
    return tiles[: 3 * n_tiles.value], items[: n_items.value]


def choose_splits(n_items: int, heads: int, kv_heads: int, longest_context: int, sms: int | None = None) -> int:
    """Splits of the keys for the token shape: about two blocks per SM of the device (``sms``, asked from the current
    device when absent) in all, at least 3 key tiles each."""
    group = heads // kv_heads
    blocks = n_items * kv_heads * ((group + 15) // 16)
    key_tiles = -(-longest_context // KEY_TILE)
    target = BLOCKS_PER_SM * (sms or sm_count())
    return max(1, min(target // max(1, blocks), key_tiles // 3, 64))


_WORK: dict[int, torch.Tensor] = {}


def work_counters(device: torch.device) -> torch.Tensor:
    """Two int32 words per device from which the persistent blocks of the tcgen05 prompt attention take their work items:
    zero between launches (the kernel's last block sets them back).  Launches on one device follow one another in one
    stream; two streams launching that kernel at once would share the counter."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _WORK:
        _WORK[index] = torch.zeros(2, dtype=torch.int32, device=torch.device("cuda", index))
    return _WORK[index]


def _common(q, out, cache, block_table, token_row, positions):
    require_cuda(q, out, cache, block_table, token_row, positions)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or q.stride(-1) != 1 or not cache.is_contiguous():
        raise KernelError("attention (bfloat16): queries and cache must be dense bfloat16")


def attention_tiles(q, heads, cache, block_table, token_row, positions, tiles, n_tiles, scale, window, out, tile_size: int = TILE_ROWS):
    """``tile_size``: the virtual rows per tile the tiles were planned for (64, or 256 for the tcgen05 kernel)."""
    _common(q, out, cache, block_table, token_row, positions)
    pages, _, kv_heads, page_size, head_dim = cache.shape
    if uses_tcgen05(head_dim, page_size) and tile_size == TC_TILE_ROWS:
        check(library("attention_tcgen05", HB_HEAD_DIM=head_dim).hb_attention_tc_tiles(
            ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table), i32(block_table.shape[1]), ptr(token_row),
            ptr(positions), ptr(tiles), i32(n_tiles), i32(q.shape[0]), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages),
            f32(scale), i32(window or 0), ptr(status_word(q.device)), ptr(work_counters(q.device)), stream_ptr()), "attention_tiles")
        return
    entry = _entry(head_dim, page_size, "tiles")
    check(entry(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table),
                                 i32(block_table.shape[1]), ptr(token_row), ptr(positions), ptr(tiles), i32(n_tiles), i32(heads),
                                 i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale), i32(window or 0),
                                 ptr(status_word(q.device)), stream_ptr()), "attention_tiles")


def attention_tokens(q, heads, cache, block_table, token_row, positions, items, n_items, splits, scale, window, out, workspace=None):
    _common(q, out, cache, block_table, token_row, positions)
    pages, _, kv_heads, page_size, head_dim = cache.shape
    if splits > 1:
        need = n_items * heads * splits * (head_dim + 2)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.float32, device=q.device)
        elif workspace.numel() < need or workspace.dtype != torch.float32:
            raise KernelError(f"attention_tokens: workspace of {need} floats needed")
    check(_entry(head_dim, page_size, "tokens")(ptr(q), i32(q.stride(0)), ptr(out), i32(out.stride(0)), ptr(cache), ptr(block_table),
                                  i32(block_table.shape[1]), ptr(token_row), ptr(positions), ptr(items), i32(n_items), i32(splits),
                                  ptr(workspace), i32(heads), i32(kv_heads), i32(head_dim), i32(page_size), i32(pages), f32(scale),
                                  i32(window or 0), ptr(status_word(q.device)), stream_ptr()), "attention_tokens")
    if splits > 1:
        from . import native

        native.LAUNCHES[0] += 1  # the merge kernel
