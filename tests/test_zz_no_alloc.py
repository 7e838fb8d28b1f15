"""The non-allocating decode-attention entry point, called through its exported C symbol.

``hb_attention_tokens_static`` is for callers that cannot allocate device memory when they call
(inside a stream capture or a latency-critical loop, plug-ins that only receive buffers, processes
with a memory budget fixed at start): the library carries the workspace of the split-key kernel in a
fixed device array.  The test checks it against the allocating entry point ``hb_attention_tokens``
on two calls in a row (the second call finds the first call's contents in the array), and that a
request larger than the array is refused without a launch.  This file sorts last on purpose.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed: int, heads=8, kv_heads=2, head_dim=64, page_size=16, contexts=(333, 65, 200)):
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page_size) for c in contexts]
    pages = sum(blocks) + 3
    order = torch.randperm(pages, generator=g).tolist()
    cache = (torch.randn(pages, 2, kv_heads, page_size, head_dim, generator=g)).to(torch.bfloat16)
    table = torch.full((len(contexts), max(blocks)), -1, dtype=torch.int32)
    for r, n in enumerate(blocks):
        for b in range(n):
            table[r, b] = order.pop()
    q = torch.randn(len(contexts), (heads + 2 * kv_heads) * head_dim, generator=g).to(torch.bfloat16)
    positions = torch.tensor([c - 1 for c in contexts], dtype=torch.int32)
    rows = torch.arange(len(contexts), dtype=torch.int32)
    return heads, kv_heads, head_dim, page_size, pages, cache.cuda(), table.cuda(), q.cuda(), positions.cuda(), rows.cuda()


def _call(function, case, splits, out, workspace=None):
    heads, kv_heads, head_dim, page_size, pages, cache, table, q, positions, rows = case
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    args = [p(q), ctypes.c_int(q.stride(0)), p(out), ctypes.c_int(out.stride(0)), p(cache), p(table), ctypes.c_int(table.shape[1]), p(rows),
            p(positions), p(rows), ctypes.c_int(q.shape[0]), ctypes.c_int(splits)]
    if workspace is not None:
        args.append(p(workspace))
    args += [ctypes.c_int(heads), ctypes.c_int(kv_heads), ctypes.c_int(head_dim), ctypes.c_int(page_size), ctypes.c_int(pages),
             ctypes.c_float(head_dim ** -0.5), ctypes.c_int(0), p(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)]
    code = function(*args)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return code


def test_static_entry_point_matches_the_allocating_one_twice_in_a_row():
    from hyperion_b200.csrc import build

    library = build.load("attention_tokens_static", {"HB_HEAD_DIM": 64})
    static, allocating = library.hb_attention_tokens_static, library.hb_attention_tokens
    library.hb_attention_tokens_static_capacity.restype = ctypes.c_longlong
    capacity = library.hb_attention_tokens_static_capacity()
    assert capacity == 4 * 1024 * 1024
    for seed, splits in ((1, 3), (2, 4)):  # two calls in a row, other inputs the second time
        case = _case(seed)
        heads, head_dim, tokens = case[0], case[2], case[7].shape[0]
        want = torch.zeros(tokens, heads * head_dim, dtype=torch.bfloat16, device="cuda")
        got = torch.ones_like(want)
        workspace = torch.empty(tokens * heads * splits * (head_dim + 2), dtype=torch.float32, device="cuda")
        assert _call(allocating, case, splits, want, workspace) == 0
        before = torch.cuda.memory_allocated()
        assert _call(static, case, splits, got) == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(got.float()).all()
        # the same kernels in the same order: the tolerance of the kernel tests (2 bf16 ulps of the largest value) is met with room
        assert (got.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()
        assert torch.equal(got, want)
    # a call that would need more than the array holds is refused, and the output is left alone
    case = _case(3)
    heads, head_dim, tokens = case[0], case[2], case[7].shape[0]
    too_many = capacity // (tokens * heads * (head_dim + 2)) + 1
    untouched = torch.full((tokens, heads * head_dim), 7.0, dtype=torch.bfloat16, device="cuda")
    assert _call(static, case, too_many, untouched) == -3
    assert bool((untouched == 7.0).all())
