"""Each kernel alone against a plain float64 computation, at sizes other than the tiny models'."""
from __future__ import annotations

import math

import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"


def ops():
    from hyperion_b200 import ops as module

    return module


def rnd(*shape, seed=0, scale=1.0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def test_embedding_copies_rows_exactly():
    for dtype in (torch.float32, torch.bfloat16):
        table = rnd(301, 72, seed=1, dtype=dtype)
        ids = torch.tensor([5, 300, 0, 17, 5], dtype=torch.int32)
        out = ops().embedding(table.to(DEV), ids.to(DEV))
        assert out.dtype == torch.float32 and torch.equal(out.cpu(), table[ids.long()].float())


def test_embedding_flags_a_bad_token_instead_of_faulting():
    from hyperion_b200.ops import KernelError, raise_on_status

    table = rnd(10, 8).to(DEV)
    ops().embedding(table, torch.tensor([3, 10], dtype=torch.int32, device=DEV))
    with pytest.raises(KernelError, match="token id"):
        raise_on_status(table.device)
    raise_on_status(table.device)  # cleared


@pytest.mark.parametrize("hidden, eps", [(72, 1e-6), (1000, 1e-5), (4104, 1e-6), (1004, 1e-6), (9000, 1e-5), (3584, 1e-6)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, eps, out_dtype):
    h = rnd(7, hidden, seed=2, scale=3.0)
    delta = rnd(7, hidden, seed=3).to(out_dtype)
    w = 1 + rnd(hidden, seed=4, scale=0.1)
    hd = h.to(DEV).clone()
    x = ops().add_rmsnorm(hd, delta.to(DEV), w.to(DEV), eps, out_dtype)
    total = h.double() + delta.double()
    want = plain.rmsnorm(total, w.double(), eps)
    assert torch.allclose(hd.cpu().double(), total, rtol=0, atol=1e-6)  # the residual stream holds the float sum
    tolerance = 2e-6 if out_dtype == torch.float32 else 2 ** -8
    assert (x.cpu().double() - want).abs().max() <= tolerance * want.abs().max()
    # without delta, and gathered rows that leave h alone
    before = hd.clone()
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    y = ops().add_rmsnorm(hd, delta.to(DEV), w.to(DEV), eps, out_dtype, rows)
    assert torch.equal(hd, before)
    want_rows = plain.rmsnorm(before.cpu().double()[rows.cpu().long()] + delta.double()[rows.cpu().long()], w.double(), eps)
    assert (y.cpu().double() - want_rows).abs().max() <= tolerance * want_rows.abs().max()
    z = ops().add_rmsnorm(hd, None, w.to(DEV), eps, out_dtype)
    want_z = plain.rmsnorm(before.cpu().double(), w.double(), eps)
    assert (z.cpu().double() - want_z).abs().max() <= tolerance * want_z.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("inter, block", [(330, None), (384, 128), (96, 24), (330, 5)])
def test_swiglu(dtype, inter, block):
    """All gate columns first, or gate and up columns alternating in runs of `block` (the layout a fused product wants)."""
    gate_up = rnd(5, 2 * inter, seed=5, scale=2.0, dtype=dtype)
    out = ops().swiglu(gate_up.to(DEV), block=block)
    runs = gate_up.double().view(5, -1, 2, block or inter)
    g, u = runs[:, :, 0].reshape(5, inter), runs[:, :, 1].reshape(5, inter)
    want = g / (1 + torch.exp(-g)) * u
    tolerance = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert (out.cpu().double() - want).abs().max() <= tolerance * want.abs().max()


def test_gate_up_with_swiglu_fused_or_not_gives_the_same_values():
    """`gated_linear` over an interleaved gate/up matrix: 700 rows take the pair kernel with SwiGLU in its epilogue, 40 rows
    the swapped product and the SwiGLU kernel; both against float64 with the projections rounded to bfloat16 first."""
    import importlib

    from hyperion_b200.ops import gemm

    routing = importlib.import_module("hyperion_b200.ops.linear")  # the module: the package's attribute of that name is the function
    inter, hidden = 384, 2048
    gate, up = rnd(inter, hidden, seed=31, scale=0.05, dtype=torch.bfloat16), rnd(inter, hidden, seed=32, scale=0.05, dtype=torch.bfloat16)
    weight = gemm.interleave_gate_up(gate.to(DEV), up.to(DEV))
    assert routing.fuses_swiglu(700, hidden) and not routing.fuses_swiglu(40, hidden) and not routing.fuses_swiglu(520, hidden)
    for rows in (700, 40):
        x = rnd(rows, hidden, seed=33, dtype=torch.bfloat16)
        got = ops().gated_linear(x.to(DEV), weight, gemm.SWIGLU_BLOCK)
        g = (x.double() @ gate.double().t()).to(torch.bfloat16).double()
        u = (x.double() @ up.double().t()).to(torch.bfloat16).double()
        want = g / (1 + torch.exp(-g)) * u
        assert (got.cpu().double() - want).abs().max() <= 2 ** -7 * want.abs().max(), rows
    plain = torch.cat([gate, up]).to(DEV)
    x = rnd(40, hidden, seed=34, dtype=torch.bfloat16).to(DEV)
    assert torch.equal(ops().gated_linear(x, plain, None), ops().gated_linear(x, weight, gemm.SWIGLU_BLOCK))  # the layout changes nothing


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim, theta", [(48, 1e4), (80, 1e6)])
def test_rope_rotates_only_the_leading_heads(dtype, head_dim, theta):
    from hyperion_b200.parts.rope import rotary_table

    heads, extra = 5, 24
    positions = torch.tensor([0, 1, 999, 37, 4095], dtype=torch.int32)
    x = rnd(5, heads * head_dim + extra, seed=6, dtype=dtype)
    table = rotary_table(head_dim, theta, 4096)
    xd = x.to(DEV).clone()
    ops().rope_(xd, heads, head_dim, positions.to(DEV), table.to(DEV))
    cos, sin = plain.rope_tables(positions, head_dim, theta)
    want = plain.rope(x.double()[:, : heads * head_dim].view(5, heads, head_dim), cos, sin).reshape(5, -1)
    tolerance = 1e-6 if dtype == torch.float32 else 2 ** -8
    got = xd.cpu().double()
    assert (got[:, : heads * head_dim] - want).abs().max() <= tolerance * want.abs().max()
    assert torch.equal(xd.cpu()[:, heads * head_dim:], x[:, heads * head_dim:])  # the rest of the row is untouched


def test_rope_flags_a_position_beyond_the_table():
    from hyperion_b200.ops import KernelError, raise_on_status
    from hyperion_b200.parts.rope import rotary_table

    x = rnd(2, 32).to(DEV)
    ops().rope_(x, 1, 32, torch.tensor([0, 64], dtype=torch.int32, device=DEV), rotary_table(32, 1e4, 64).to(DEV))
    with pytest.raises(KernelError, match="position"):
        raise_on_status(x.device)


@pytest.mark.parametrize("m", [1, 3, 64, 130])
def test_sgemm_f32_matches_float64_and_does_not_depend_on_the_batch(m):
    k, n = 331, 203
    x, w, b = rnd(130, k, seed=7), rnd(n, k, seed=8), rnd(n, seed=9)
    full = ops().sgemm_f32(x.to(DEV), w.to(DEV), b.to(DEV)).cpu()
    want = x.double() @ w.double().t() + b.double()
    assert (full.double() - want).abs().max() <= 2e-6 * want.abs().max() * math.sqrt(k)
    part = ops().sgemm_f32(x[:m].to(DEV), w.to(DEV), b.to(DEV)).cpu()
    assert torch.equal(part, full[:m])  # bit for bit: a row's result does not depend on its neighbours
    strided = x.to(DEV)[:, : k - 3]
    got = ops().sgemm_f32(strided, w[:, : k - 3].contiguous().to(DEV)).cpu()
    assert torch.allclose(got.double(), x.double()[:, : k - 3] @ w.double()[:, : k - 3].t(), atol=1e-4)


def paged_case(kv_heads, head_dim, page_size, contexts, dtype, seed=0, pages_extra=5):
    """Random keys/values for requests of the given context lengths scattered over shuffled pages."""
    g = torch.Generator().manual_seed(seed)
    blocks = [-(-c // page_size) for c in contexts]
    pages = sum(blocks) + pages_extra
    order = torch.randperm(pages, generator=g).tolist()
    cache = torch.full((pages, 2, kv_heads, page_size, head_dim), float("nan"), dtype=dtype)  # pages nobody holds are NaN
    width = max(blocks) + 2
    table = torch.full((len(contexts), width), -1, dtype=torch.int32)
    keys, values = [], []
    for r, c in enumerate(contexts):
        k = rnd(c, kv_heads, head_dim, seed=seed * 100 + 2 * r, dtype=dtype)
        v = rnd(c, kv_heads, head_dim, seed=seed * 100 + 2 * r + 1, dtype=dtype)
        keys.append(k)
        values.append(v)
        for b in range(blocks[r]):
            page = order.pop()
            table[r, b] = page
            n = min(page_size, c - b * page_size)
            cache[page, 0, :, :n] = k[b * page_size : b * page_size + n].transpose(0, 1)
            cache[page, 1, :, :n] = v[b * page_size : b * page_size + n].transpose(0, 1)
            # slots of a held page past the context: in the engine they hold what the page's last owner left there, finite
            # keys and values of any size; a kernel that lets one of them into a sum is off by far more than the tolerance
            sign = torch.where(torch.rand((2, kv_heads, page_size - n, head_dim), generator=g) < 0.5, -1.0, 1.0)
            cache[page, :, :, n:] = (sign * 300.0).to(dtype)
    return cache, table, keys, values


def test_kv_store_writes_where_the_table_says_and_nowhere_else():
    kv_heads, head_dim, page_size = 3, 16, 8
    cache = torch.zeros(6, 2, kv_heads, page_size, head_dim)
    table = torch.tensor([[4, 1, -1], [2, 5, 0]], dtype=torch.int32)
    token_row = torch.tensor([0, 0, 1, 1, 1], dtype=torch.int32)
    positions = torch.tensor([7, 8, 15, 16, 17], dtype=torch.int32)
    width = kv_heads * head_dim
    src = rnd(5, 10 + 2 * width, seed=11)
    cd = cache.to(DEV)
    ops().kv_store(src.to(DEV), 10, 10 + width, cd, table.to(DEV), token_row.to(DEV), positions.to(DEV))
    want = cache.clone()
    for t in range(5):
        page = table[token_row[t], positions[t] // page_size]
        slot = positions[t] % page_size
        want[page, 0, :, slot] = src[t, 10 : 10 + width].view(kv_heads, head_dim)
        want[page, 1, :, slot] = src[t, 10 + width :].view(kv_heads, head_dim)
    assert torch.equal(cd.cpu(), want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("head_dim", [24, 32, 128])  # 32 and 128 take the 16-byte variant in bfloat16
def test_fused_rope_and_cache_write_equals_the_two_steps(dtype, head_dim):
    from hyperion_b200.parts.rope import rotary_table

    q_heads, kv_heads, page_size = 5, 3, 4
    table = torch.tensor([[2, 0, 5, -1], [1, 3, 4, 6]], dtype=torch.int32).to(DEV)
    token_row = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32).to(DEV)
    positions = torch.tensor([3, 4, 11, 0, 15], dtype=torch.int32).to(DEV)
    rope_table = rotary_table(head_dim, 1e4, 64).to(DEV)
    x = rnd(5, (q_heads + 2 * kv_heads) * head_dim, seed=21, dtype=dtype).to(DEV)
    a, b = x.clone(), x.clone()
    cache_a = torch.zeros(7, 2, kv_heads, page_size, head_dim, dtype=dtype, device=DEV)
    cache_b = cache_a.clone()
    ops().rope_(a, q_heads + kv_heads, head_dim, positions, rope_table)
    ops().kv_store(a, q_heads * head_dim, (q_heads + kv_heads) * head_dim, cache_a, table, token_row, positions)
    ops().rope_kv_store_(b, q_heads, kv_heads, head_dim, positions, rope_table, cache_b, table, token_row)
    assert torch.equal(cache_a, cache_b)
    assert torch.equal(a[:, : q_heads * head_dim], b[:, : q_heads * head_dim])
    assert torch.equal(b[:, q_heads * head_dim:], x[:, q_heads * head_dim:])  # the row's own k and v are left alone


def reference_attention(q, keys, values, rows, scale, window):
    """q [T, heads, d] float64; rows: list of (request index, first position, count)."""
    outs = []
    at = 0
    for request, first, count in rows:
        k, v = keys[request].double(), values[request].double()
        qp = torch.arange(first, first + count)
        kp = torch.arange(k.shape[0])
        outs.append(plain.attention(q[at : at + count], k, v, qp, kp, scale, window))
        at += count
    return torch.cat(outs)


@pytest.mark.parametrize("heads, kv_heads, head_dim, page_size, window", [(6, 2, 24, 8, 0), (5, 5, 40, 16, 0), (20, 2, 16, 4, 0), (4, 1, 72, 32, 37)])
def test_attention_generic_float32(heads, kv_heads, head_dim, page_size, window):
    contexts = [150, 9, 77]
    cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, contexts, torch.float32, seed=3)
    rows = [(0, 150 - 20, 20), (1, 8, 1), (2, 0, 77)]
    tokens = sum(r[2] for r in rows)
    q = rnd(tokens, heads * head_dim + 8, seed=12)
    token_row = torch.tensor([i for i, r in enumerate(rows) for _ in range(r[2])], dtype=torch.int32)
    positions = torch.tensor([p for r in rows for p in range(r[1], r[1] + r[2])], dtype=torch.int32)
    scale = head_dim ** -0.5
    out = ops().attention_generic(q.to(DEV), heads, cache.to(DEV), table.to(DEV), token_row.to(DEV), positions.to(DEV), scale, window)
    want = reference_attention(q[:, : heads * head_dim].double().view(tokens, heads, head_dim), keys, values, rows, scale, window)
    assert (out.cpu().double().view(tokens, heads, head_dim) - want).abs().max() <= 5e-6 * want.abs().max()
    # one token alone gives the same bits as inside the batch
    pick = 25
    alone = ops().attention_generic(q[pick : pick + 1].to(DEV), heads, cache.to(DEV), table.to(DEV), token_row[pick : pick + 1].to(DEV),
                                    positions[pick : pick + 1].to(DEV), scale, window)
    assert torch.equal(alone.cpu()[0], out.cpu()[pick])


def run_fast_attention(q, heads, cache, table, rows, scale, window):
    from hyperion_b200.engine.batch import Row
    from hyperion_b200.ops import attention as fast

    kv_heads = cache.shape[2]
    step_rows, start = [], 0
    for i, (request, first, count) in enumerate(rows):
        step_rows.append(Row(request, start, count, first, i))
        start += count
    tiles, items = (a.tolist() for a in fast.plan(step_rows, fast.tile_tokens(heads, kv_heads)))
    token_row = torch.tensor([i for i, r in enumerate(rows) for _ in range(r[2])], dtype=torch.int32, device=DEV)
    positions = torch.tensor([p for r in rows for p in range(r[1], r[1] + r[2])], dtype=torch.int32, device=DEV)
    batch_table = table[[r[0] for r in rows]].contiguous().to(DEV)
    out = torch.full((q.shape[0], heads * cache.shape[-1]), float("nan"), dtype=torch.bfloat16, device=DEV)
    qd, cd = q.to(DEV), cache.to(DEV)
    if tiles:
        fast.attention_tiles(qd, heads, cd, batch_table, token_row, positions, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             len(tiles) // 3, scale, window, out)
    outs = {}
    page_size, head_dim = cache.shape[3], cache.shape[4]
    if tiles and fast.uses_tcgen05(head_dim, page_size):  # the same rows again through the tcgen05 kernel (256-row tiles)
        wide = fast.plan(step_rows, fast.tile_tokens(heads, kv_heads, fast.TC_TILE_ROWS))[0].tolist()
        o = out.clone()
        fast.attention_tiles(qd, heads, cd, batch_table, token_row, positions, torch.tensor(wide, dtype=torch.int32, device=DEV),
                             len(wide) // 3, scale, window, o, tile_size=fast.TC_TILE_ROWS)
        if items:
            fast.attention_tokens(qd, heads, cd, batch_table, token_row, positions, torch.tensor(items, dtype=torch.int32, device=DEV),
                                  len(items), 2, scale, window, o)
        outs["tcgen05"] = o
    if items:
        items_dev = torch.tensor(items, dtype=torch.int32, device=DEV)
        # 9 and 40 splits leave splits without keys
        for splits in (1, 3, 9, 40):
            o = out.clone()
            fast.attention_tokens(qd, heads, cd, batch_table, token_row, positions, items_dev, len(items), splits, scale, window, o)
            again = out.clone()
            fast.attention_tokens(qd, heads, cd, batch_table, token_row, positions, items_dev, len(items), splits, scale, window, again)
            assert torch.equal(o.view(torch.int16), again.view(torch.int16)), f"splits {splits}: a second launch gives other bits"
            outs[splits] = o
    else:
        outs[1] = out
    return outs


@pytest.mark.parametrize("heads, kv_heads, head_dim, page_size, window", [(14, 2, 64, 16, 0), (6, 1, 32, 8, 0), (8, 8, 80, 16, 0),
                                                                          (20, 1, 16, 4, 0), (4, 2, 128, 32, 100), (3, 1, 48, 16, 70),
                                                                          (28, 4, 128, 16, 0), (4, 1, 64, 64, 0), (4, 2, 192, 8, 50),
                                                                          (36, 2, 64, 16, 0), (130, 1, 64, 16, 0), (264, 1, 64, 16, 0)])
def test_attention_bf16_tiles_and_tokens(heads, kv_heads, head_dim, page_size, window):
    from hyperion_b200.ops import raise_on_status

    contexts = [300, 9, 130, 64, 513]
    cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, contexts, torch.bfloat16, seed=5)
    rows = [(0, 300 - 70, 70), (1, 8, 1), (2, 0, 130), (3, 62, 2), (4, 512, 1), (0, 0, 0)][:5]
    tokens = sum(r[2] for r in rows)
    q = rnd(tokens, (heads + 2 * kv_heads) * head_dim, seed=13, dtype=torch.bfloat16)
    scale = head_dim ** -0.5
    outs = run_fast_attention(q, heads, cache, table, rows, scale, window)
    raise_on_status(torch.device(DEV))
    want = reference_attention(q[:, : heads * head_dim].double().view(tokens, heads, head_dim), keys, values, rows, scale, window)
    for splits, out in outs.items():
        got = out.cpu().double().view(tokens, heads, head_dim)
        assert torch.isfinite(got).all(), f"splits {splits}: not finite"
        assert (got - want).abs().max() <= 2 ** -7 * want.abs().max(), f"splits {splits}"


def test_prompt_attention_with_more_short_items_than_blocks():
    """Hundreds of short prompt portions in one launch: every persistent block of the tcgen05 kernel takes several
    items one after the other, most of them a single tile of keys (the next item's queries are then wanted before the
    softmax threads have looked at this item's), some of two or three, some that run one half of the block alone."""
    from hyperion_b200.ops import raise_on_status

    heads, kv_heads, head_dim, page_size = 8, 2, 128, 16
    g = torch.Generator().manual_seed(77)
    counts = torch.randint(5, 70, (360,), generator=g).tolist()
    firsts = [int(f) for f in torch.randint(0, 300, (360,), generator=g)]
    for i in range(0, 360, 9):
        firsts[i] = 0  # whole short prompts among the portions
    contexts = [f + c for f, c in zip(firsts, counts)]
    cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, contexts, torch.bfloat16, seed=8)
    rows = [(r, firsts[r], counts[r]) for r in range(360)]
    tokens = sum(counts)
    q = rnd(tokens, (heads + 2 * kv_heads) * head_dim, seed=15, dtype=torch.bfloat16)
    scale = head_dim ** -0.5
    outs = run_fast_attention(q, heads, cache, table, rows, scale, 0)
    raise_on_status(torch.device(DEV))
    want = reference_attention(q[:, : heads * head_dim].double().view(tokens, heads, head_dim), keys, values, rows, scale, None)
    got = outs["tcgen05"].cpu().double().view(tokens, heads, head_dim)
    assert torch.isfinite(got).all()
    assert (got - want).abs().max() <= 2 ** -7 * want.abs().max()


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_prompt_attention_of_random_shapes(seed):
    """Ten random steps per seed (head size 64 or 128, 1 to 8 key/value heads with 1 to 18 query heads each, pages of 8 to
    64, with and without a window, 1 to 30 portions of 5 to 900 tokens at positions up to 3,000) through the tcgen05
    kernel, each against the plain attention in float64."""
    import random

    from hyperion_b200.engine.batch import Row
    from hyperion_b200.ops import attention as fast
    from hyperion_b200.ops import raise_on_status

    rng = random.Random(seed)
    for case in range(10):
        head_dim, kv_heads, group = rng.choice([64, 128]), rng.choice([1, 2, 4, 8]), rng.choice([1, 2, 3, 4, 7, 8, 16, 18])
        heads, page_size = kv_heads * group, rng.choice([8, 16, 32, 64])
        window = rng.choice([0, 0, rng.randrange(1, 600)])
        n_rows = rng.randrange(1, 30)
        counts = [rng.choice([rng.randrange(5, 40), rng.randrange(5, 300), rng.randrange(5, 900)]) for _ in range(n_rows)]
        firsts = [rng.choice([0, rng.randrange(0, 200), rng.randrange(0, 3000)]) for _ in range(n_rows)]
        cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, [f + c for f, c in zip(firsts, counts)], torch.bfloat16,
                                                seed=100 * seed + case)
        tokens = sum(counts)
        q = rnd(tokens, (heads + 2 * kv_heads) * head_dim, seed=1000 + 100 * seed + case, dtype=torch.bfloat16).to(DEV)
        rows, at = [], 0
        for i, (first, count) in enumerate(zip(firsts, counts)):
            rows.append(Row(i, at, count, first, i))
            at += count
        size = fast.TC_TILE_ROWS
        tiles = fast.plan(rows, fast.tile_tokens(heads, kv_heads, size))[0]
        token_row = torch.tensor([i for i, c in enumerate(counts) for _ in range(c)], dtype=torch.int32, device=DEV)
        positions = torch.tensor([p for f, c in zip(firsts, counts) for p in range(f, f + c)], dtype=torch.int32, device=DEV)
        out = torch.full((tokens, heads * head_dim), float("nan"), dtype=torch.bfloat16, device=DEV)
        fast.attention_tiles(q, heads, cache.to(DEV), table.to(DEV), token_row, positions, torch.tensor(tiles, dtype=torch.int32, device=DEV),
                             len(tiles) // 3, head_dim ** -0.5, window, out, tile_size=size)
        raise_on_status(torch.device(DEV))
        got = out.double().view(tokens, heads, head_dim)
        what = dict(case=case, head_dim=head_dim, kv_heads=kv_heads, group=group, page_size=page_size, window=window, rows=n_rows)
        assert torch.isfinite(got).all(), what
        at = 0
        for i, (first, count) in enumerate(zip(firsts, counts)):  # the plain attention in float64, on the device: the sizes are not small
            k, v = keys[i].to(DEV).double(), values[i].to(DEV).double()
            want = plain.attention(q[at : at + count, : heads * head_dim].double().view(count, heads, head_dim), k, v,
                                   torch.arange(first, first + count, device=DEV), torch.arange(k.shape[0], device=DEV), head_dim ** -0.5,
                                   window or None)
            error = (got[at : at + count] - want).abs().max() / want.abs().max()
            assert error <= 2 ** -7, (what, i, first, count, float(error))
            at += count


def test_attention_bf16_finds_one_far_key_among_hundreds():
    """Random scores would average a lost key away: make one distant key dominate every query."""
    heads, kv_heads, head_dim, page_size = 8, 2, 64, 16
    contexts = [700, 700]
    cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, contexts, torch.bfloat16, seed=6)
    for far in (3, 64 * 5 + 63, 699 - 64):  # near the start, at a tile's edge, in the last full tile
        k = [x.clone() for x in keys]
        direction = rnd(head_dim, seed=far).to(torch.bfloat16)
        c = cache.clone()
        for r in range(2):
            k[r][far] = direction * 4
            c[table[r, far // page_size], 0, :, far % page_size] = direction * 4
        rows = [(0, 650, 50), (1, 699, 1)]
        tokens = 51
        q = (direction.float() * 4).repeat(tokens, heads + 2 * kv_heads).to(torch.bfloat16)
        outs = run_fast_attention(q, heads, c, table, rows, head_dim ** -0.5, 0)
        want = reference_attention(q[:, : heads * head_dim].double().view(tokens, heads, head_dim), k, values, rows, head_dim ** -0.5, None)
        for out in outs.values():
            got = out.cpu().double().view(tokens, heads, head_dim)
            assert (got - want).abs().max() <= 2 ** -7 * want.abs().max()
            # the output is essentially the far key's value
            assert (got[0, 0] - values[0][far, 0].double()).abs().max() < 0.05


@pytest.mark.parametrize("vocab", [523, 152064])
def test_sampler_greedy_ties_and_nan(vocab):
    from hyperion_b200.sampling import GREEDY, Sampler, pack_options

    logits = rnd(4, vocab, seed=14)
    logits[0, [7, 300]] = 9.0  # a tie: the lower index wins
    logits[1, 5] = float("nan")
    logits[1, 400] = 8.0
    logits[2] = float("-inf")
    logits[2, vocab - 1] = -5.0
    sampler = Sampler(vocab, torch.device(DEV))
    options = torch.tensor([pack_options(GREEDY, 0, -1) for _ in range(4)], dtype=torch.int32, device=DEV)
    got = sampler.sample(logits.to(DEV), options).cpu().tolist()
    assert got[:3] == [7, 400, vocab - 1] and got[3] == int(torch.argmax(logits[3]))
    spread = sampler.sample(logits.to(DEV), options, all_greedy=True).cpu().tolist()  # the many-blocks-per-row argmax
    assert spread == got
    logits[0, [vocab - 2, 3]] = 11.0  # a tie across two blocks' slices
    assert sampler.sample(logits.to(DEV), options, all_greedy=True).cpu().tolist()[0] == 3


@pytest.mark.parametrize("vocab, params", [
    (523, dict(temperature=0.8)), (523, dict(temperature=1.3, top_k=40)), (523, dict(temperature=0.7, top_p=0.9)),
    (523, dict(temperature=1.0, top_k=50, top_p=0.5, repetition_penalty=1.3)), (152064, dict(temperature=0.8, top_k=50, top_p=0.95)),
    (152064, dict(temperature=1.0)), (1000, dict(temperature=1.0, top_k=1)),
    (152064, dict(temperature=0.9, top_p=0.8)), (152064, dict(temperature=1.1, top_k=3000, top_p=0.9, repetition_penalty=1.1)),
    (5000, dict(temperature=0.6, top_k=1024)), (5000, dict(temperature=0.6, top_k=1025, top_p=0.3)),
])
def test_sampler_matches_the_host_rule(vocab, params):
    """The device token must be the host reference's token, or the draw must lie within float rounding
    of the boundary between the two (the device sums in float, the reference in double)."""
    import numpy as np

    from hyperion_b200.sampling import Sampler, SamplingParams, pack_options, reference_sample

    rows = 48
    logits = rnd(rows, vocab, seed=15, scale=3.0)
    logits[:, 11] = logits[:, 12]  # ties inside the candidate set
    sampling = SamplingParams(seed=1234567890123, **params).validated()
    generated = [3, 11, 77, 500]
    seen = torch.zeros(rows, (vocab + 31) // 32, dtype=torch.int32)
    for token in generated:
        seen[:, token // 32] |= 1 << (token % 32)
    sampler = Sampler(vocab, torch.device(DEV), seen=seen.to(DEV))
    options = torch.tensor([pack_options(sampling, step, step) for step in range(rows)], dtype=torch.int32, device=DEV)
    got = sampler.sample(logits.to(DEV), options).cpu().tolist()
    exact = 0
    for row in range(rows):
        token, info = reference_sample(logits[row].numpy(), sampling, row, generated)
        if got[row] == token:
            exact += 1
            continue
        kept = info["kept"].tolist()
        assert got[row] in kept, f"row {row}: device token {got[row]} is outside the kept set"
        j = kept.index(got[row])
        lower = info["cdf"][j - 1] if j else 0.0
        assert lower - 1e-5 <= info["u"] <= info["cdf"][j] + 1e-5, f"row {row}: draw {info['u']} does not select token {got[row]}"
    assert exact >= rows - 2
    # the chosen tokens are recorded in the per-request bitmaps
    bitmap = sampler.seen.cpu()
    assert all((int(bitmap[row, got[row] // 32]) >> (got[row] % 32)) & 1 for row in range(rows))


@pytest.mark.parametrize("params, allowed", [
    (dict(temperature=1.0, top_k=3), {2, 5, 9}),             # 2 and 5 stand above; of the four equal ones the lowest index completes the three
    (dict(temperature=1.0, top_k=5), {2, 5, 9, 40, 41}),
    (dict(temperature=1.0, top_p=0.6), {2, 5, 9}),           # masses e^2, e^2, then e^1 each: six tenths of the whole need the first tie
    (dict(temperature=1.0, top_k=2000, top_p=0.6), {2, 5, 9}),
    (dict(temperature=1.0, top_k=4, top_p=0.99), {2, 5, 9, 40}),
])
def test_sampler_cuts_ties_at_the_lowest_indices(params, allowed):
    """Equal logits at the edge of the top-k set or of the nucleus: the ones with the lowest indices stay. Over many
    draws every allowed token comes up and no other does."""
    from hyperion_b200.sampling import Sampler, SamplingParams, pack_options

    vocab, draws = 3000, 600
    logits = torch.full((1, vocab), -20.0)
    logits[0, [2, 5]] = 2.0
    logits[0, [9, 40, 41, 2999]] = 1.0
    sampling = SamplingParams(seed=77, **params).validated()
    sampler = Sampler(vocab, torch.device(DEV))
    options = torch.tensor([pack_options(sampling, step, -1) for step in range(draws)], dtype=torch.int32, device=DEV)
    got = set(sampler.sample(logits.expand(draws, vocab).contiguous().to(DEV), options).cpu().tolist())
    assert got == allowed


def test_sampler_rows_of_equal_logits_and_of_nan():
    from hyperion_b200.sampling import Sampler, SamplingParams, pack_options

    vocab = 70000
    logits = torch.zeros(3, vocab)
    logits[1] = float("nan")
    logits[2] = float("nan")
    logits[2, 31] = 0.5
    sampler = Sampler(vocab, torch.device(DEV))
    for params in (dict(temperature=1.0, top_k=7), dict(temperature=1.0, top_p=0.0001), dict(temperature=1.0, top_k=7, top_p=0.5)):
        sampling = SamplingParams(seed=3, **params).validated()
        options = torch.tensor([pack_options(sampling, step, -1) for step in range(3)], dtype=torch.int32, device=DEV)
        got = sampler.sample(logits.to(DEV), options).cpu().tolist()
        assert 0 <= got[0] < 7, (params, got)   # equal everywhere: only the lowest indices are kept
        assert got[1] == 0 and got[2] == 31, (params, got)


def test_sampler_frequencies_follow_the_softmax():
    import numpy as np

    from hyperion_b200.sampling import Sampler, SamplingParams, pack_options

    vocab, draws = 16, 4000
    logits = torch.tensor([[2.0, 1.0, 0.5, 0.0, -1.0] + [-3.0] * 11])
    sampling = SamplingParams(temperature=1.0, seed=99).validated()
    sampler = Sampler(vocab, torch.device(DEV))
    options = torch.tensor([pack_options(sampling, step, -1) for step in range(draws)], dtype=torch.int32, device=DEV)
    got = sampler.sample(logits.expand(draws, vocab).contiguous().to(DEV), options).cpu().numpy()
    observed = np.bincount(got, minlength=vocab)
    expected = torch.softmax(logits[0].double(), 0).numpy() * draws
    chi2 = float(((observed - expected) ** 2 / expected).sum())
    assert chi2 < 45.0  # 15 degrees of freedom: p = 0.0001 at 42.6... a wrong sampler lands in the hundreds


@pytest.mark.parametrize("kind", ["float32", "bfloat16"])
def test_attention_at_the_edges_of_window_page_and_tile(kind):
    """One key is made to dominate (its score stands far above the rest) and placed just inside the window, just
    outside it, on the last slot of a page and on the first slot of the next, at a key tile's edge: the output must be
    that key's value when it is visible and must not contain it when it is not."""
    heads, kv_heads, head_dim, page_size, window = 4, 2, 64, 16, 40
    dtype = torch.float32 if kind == "float32" else torch.bfloat16
    context = 200
    query_pos = context - 1
    direction = rnd(head_dim, seed=31).to(dtype)
    for spot, visible in ((query_pos - window + 1, True), (query_pos - window, False), (175, True), (176, True), (191, True), (192, True),
                          (query_pos, True), (query_pos - window - 17, False)):
        cache, table, keys, values = paged_case(kv_heads, head_dim, page_size, [context], dtype, seed=9)
        keys[0][spot] = direction * 4
        cache[table[0, spot // page_size], 0, :, spot % page_size] = direction * 4
        rows = [(0, query_pos - 5, 6)] if spot % 2 else [(0, query_pos, 1)]  # a short portion (tile shape) or one token
        tokens = rows[0][2]
        q = (direction.float() * 4).repeat(tokens, heads + 2 * kv_heads).to(dtype)
        scale = head_dim ** -0.5
        if kind == "float32":
            token_row = torch.zeros(tokens, dtype=torch.int32)
            positions = torch.arange(rows[0][1], rows[0][1] + tokens, dtype=torch.int32)
            out = ops().attention_generic(q.to(DEV), heads, cache.to(DEV), table.to(DEV), token_row.to(DEV), positions.to(DEV), scale, window)
            outs = {1: out}
        else:
            outs = run_fast_attention(q, heads, cache, table, rows, scale, window)
        want = reference_attention(q[:, : heads * head_dim].double().view(tokens, heads, head_dim), keys, values, rows, scale, window)
        for out in outs.values():
            got = out.cpu().double().view(tokens, heads, head_dim)
            assert (got - want).abs().max() <= (1e-5 if kind == "float32" else 2 ** -7) * want.abs().max(), (spot, visible)
            distance = (got[-1, 0] - values[0][spot, 0].double()).abs().max()
            assert (distance < 0.05) == visible, (spot, visible, float(distance))


@pytest.mark.parametrize("tokens, hidden, splits, with_rows", [(8, 3584, 5, False), (3, 72, 2, False), (33, 9000, 3, True), (64, 1000, 7, True)])
def test_norm_that_adds_up_split_sums_itself_gives_the_bits_of_the_two_kernel_path(tokens, hidden, splits, with_rows):
    """The delta arrives as split-K pieces: adding them up inside the norm kernel equals adding them up first."""
    from hyperion_b200.ops.gemm import SplitSum

    partials = rnd(splits, tokens, hidden, seed=40).to(DEV)
    bias = rnd(hidden, seed=41).to(torch.bfloat16).to(DEV)
    w = (1 + rnd(hidden, seed=42, scale=0.1)).to(DEV)
    rows = torch.tensor([tokens - 1, 0], dtype=torch.int32, device=DEV) if with_rows else None
    for b in (bias, bias.float(), None):
        h1, h2 = rnd(tokens, hidden, seed=43, scale=3.0).to(DEV), rnd(tokens, hidden, seed=43, scale=3.0).to(DEV)
        pieces = SplitSum(partials, b, torch.bfloat16)
        fused = ops().add_rmsnorm(h1, pieces, w, 1e-6, torch.bfloat16, rows)
        plain_way = ops().add_rmsnorm(h2, pieces.tensor(), w, 1e-6, torch.bfloat16, rows)
        assert torch.equal(fused, plain_way) and torch.equal(h1, h2)
    total = partials.double().sum(0) + bias.double()
    assert (pieces.tensor().double() - partials.double().sum(0)).abs().max() <= 2 ** -8 * total.abs().max() + 1e-3


@pytest.mark.parametrize("heads, kv_heads, head_dim", [(36, 2, 64), (28, 4, 128)])
def test_attention_gives_the_same_bits_every_time(heads, kv_heads, head_dim):
    """Races show as results that change from run to run: the same launches 60 times over, with freed memory
    overwritten by NaN in between so that anything read before it is written shows too."""
    contexts = [300, 9, 130, 64, 513]
    cache, table, keys, values = paged_case(kv_heads, head_dim, 16, contexts, torch.bfloat16, seed=5)
    rows = [(0, 300 - 70, 70), (1, 8, 1), (2, 0, 130), (3, 62, 2), (4, 512, 1)]
    tokens = sum(r[2] for r in rows)
    q = rnd(tokens, (heads + 2 * kv_heads) * head_dim, seed=13, dtype=torch.bfloat16)
    first = None
    for _ in range(60):
        poison = [torch.full((n,), float("nan"), device=DEV) for n in (1 << 12, 1 << 16, 1 << 20, 1 << 24)]
        del poison
        outs = {k: v.cpu() for k, v in run_fast_attention(q, heads, cache, table, rows, head_dim ** -0.5, 0).items()}
        if first is None:
            first = outs
        for key, value in outs.items():
            assert torch.equal(value, first[key]), f"variant {key} changed between runs"
