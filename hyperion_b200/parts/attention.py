"""Causal grouped-query attention over the paged cache.

Per step: one fused projection to [q | k | v] with bias, position encoding of q and k in place, the
new keys and values written to their pages, then attention of every token over its request's
cache, and the output projection.  The order is the reference's: the cache is written before
attention reads it (helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:716-772); q, k and v
share one [Q+2KV, H] matrix placed back to back at load (backend.rs:95-106); query head h reads
key/value head h // (heads / kv_heads) and sees keys at positions <= its own
(helios/crates/helios-hal/src/reference.rs:118-156).

Parameters: ``hidden_size``, ``heads``, ``kv_heads``, ``head_dim``, ``bias`` (on q, k, v),
``scale`` (default head_dim**-0.5), ``window`` (0 = all keys), ``position`` (a PartSpec or None),
``shares_kv`` (true: the part owns no k/v projection and only reads the cache it is given).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..ops import attention as fast_attention
from .base import POSITIONS, BuildContext, Mixer, PagedKV, WeightSpec, make, register_mixer
from .spec import PartSpec


def _common_dtype(tensors) -> torch.dtype:
    return torch.float32 if any(t.dtype == torch.float32 for t in tensors) else tensors[0].dtype


class GroupedQueryAttention(Mixer):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.kv_heads = int(p["kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.bias = bool(p.get("bias", False))
        self.scale = float(p.get("scale", self.head_dim ** -0.5))
        self.window = int(p.get("window", 0) or 0)
        self.shares_kv = bool(p.get("shares_kv", False))
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.kv_heads} key/value heads do not divide {self.heads} heads")
        if self.head_dim > 256:
            raise ValueError(f"head_dim {self.head_dim} is above the kernels' limit of 256")
        self.position = make(POSITIONS, p["position"], build) if p.get("position") is not None else None
        self.q_width = self.heads * self.head_dim
        self.kv_width = self.kv_heads * self.head_dim
        # the tensor-core kernels take bfloat16 and head sizes in steps of 16; other head sizes use the generic kernel
        self.fast = self.dtype == torch.bfloat16 and fast_attention.supported(self.head_dim)

    def weights(self) -> dict[str, WeightSpec]:
        names = {"q_proj.weight": WeightSpec((self.q_width, self.hidden)), "o_proj.weight": WeightSpec((self.hidden, self.q_width))}
        if not self.shares_kv:
            names["k_proj.weight"] = WeightSpec((self.kv_width, self.hidden))
            names["v_proj.weight"] = WeightSpec((self.kv_width, self.hidden))
        if self.bias:
            names["q_proj.bias"] = WeightSpec((self.q_width,))
            if not self.shares_kv:
                names["k_proj.bias"] = WeightSpec((self.kv_width,))
                names["v_proj.bias"] = WeightSpec((self.kv_width,))
        return names

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        order = ["q_proj"] if self.shares_kv else ["q_proj", "k_proj", "v_proj"]
        mats = [tensors[f"{n}.weight"] for n in order]
        dtype = _common_dtype(mats)
        self.w_qkv = torch.cat([m.to(dtype) for m in mats], dim=0).contiguous()
        self.b_qkv = torch.cat([tensors[f"{n}.bias"].to(dtype) for n in order], dim=0).contiguous() if self.bias else None
        self.w_o = tensors["o_proj.weight"].contiguous()

    def cache_request(self):
        return None if self.shares_kv else PagedKV(self.kv_heads, self.head_dim, self.window)

    def kernel_modules(self):
        modules = [("elementwise", {})]
        if self.fast:  # which of the two is launched depends on the page size of the cache it is given
            modules.append(("attention_bf16", {"HB_HEAD_DIM": self.head_dim}))
            if self.head_dim % 64 == 0:
                modules.append(("attention_tma", {"HB_HEAD_DIM": self.head_dim}))
            if self.head_dim in (64, 128):
                modules.append(("attention_tcgen05", {"HB_HEAD_DIM": self.head_dim}))
        else:
            modules.append(("attention_generic", {}))
        modules.append(("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {}))
        if self.position is not None:
            modules += self.position.kernel_modules()
        return modules

    def forward(self, x, step, cache, own_cache):
        if cache is None:
            raise ValueError("attention needs a paged cache; the schedule gave it none")
        qkv = ops.linear(x, self.w_qkv, self.b_qkv, self.dtype)
        stores = own_cache and not self.shares_kv
        if self.position is not None and stores:
            self.position.apply_and_store_(qkv, self.heads, self.kv_heads, self.head_dim, step.positions, cache, step.token_row)
        else:
            if self.position is not None:
                self.position.apply_(qkv, self.heads if self.shares_kv else self.heads + self.kv_heads, self.head_dim, step.positions)
            if stores:
                ops.kv_store(qkv, self.q_width, self.q_width + self.kv_width, cache.kv, cache.block_table, step.token_row, step.positions)
        if self.fast:
            attn = self._attend_fast(qkv, step, cache)
        else:
            attn = ops.attention_generic(qkv, self.heads, cache.kv, cache.block_table, step.token_row, step.positions, self.scale, self.window)
        return ops.linear(attn, self.w_o, None, self.dtype, may_leave_partials=True)  # the result is a residual delta

    # ------------------------------------------------------------------ the tensor-core path
    def step_plans(self):
        """Per-step metadata: the rows cut into tiles and single tokens (shared by all layers with the same tiling)."""
        if not self.fast:
            return {}
        heads, kv_heads, head_dim = self.heads, self.kv_heads, self.head_dim

        def plan(rows, packer, host):
            size = fast_attention.tile_rows(head_dim, host.get("page_size"))
            tokens_per_tile = fast_attention.tile_tokens(heads, kv_heads, size)
            key = f"attn_tiles_{tokens_per_tile}"
            if key in host:
                return
            tiles, items = fast_attention.plan(rows, tokens_per_tile)
            host[key] = len(tiles) // 3
            host["attn_items"] = len(items)
            if len(tiles):
                packer.add(key, tiles)
            if len(items) and "attn_items" not in [name for name, *_ in packer._items]:
                packer.add("attn_items", items)

        return {("attention_plan", heads // kv_heads, head_dim): plan}

    @staticmethod
    def _longest_short_row(rows) -> int:
        """The largest context among the rows that go token by token."""
        if hasattr(rows, "counts"):
            short = rows.counts <= fast_attention.TOKEN_SHAPE_MAX
            return int((rows.positions[short] + rows.counts[short]).max())
        return max(row.position + row.count for row in rows if row.count <= fast_attention.TOKEN_SHAPE_MAX)

    def _attend_fast(self, qkv, step, cache):
        out = torch.empty((step.n_tokens, self.q_width), dtype=self.dtype, device=qkv.device)
        size = fast_attention.tile_rows(self.head_dim, step.host.get("page_size"))
        key = f"attn_tiles_{fast_attention.tile_tokens(self.heads, self.kv_heads, size)}"
        n_tiles, n_items = step.host.get(key, 0), step.host.get("attn_items", 0)
        if n_tiles:
            fast_attention.attention_tiles(qkv, self.heads, cache.kv, cache.block_table, step.token_row, step.positions,
                                           step.extra[key], n_tiles, self.scale, self.window, out, tile_size=size)
        if n_items:
            # a step replayed from a CUDA graph fixes its launch shape for every context its tables can hold
            longest = step.host.get("context_cap") or self._longest_short_row(step.rows)
            if self.window:
                longest = min(longest, self.window + fast_attention.KEY_TILE)
            splits = fast_attention.choose_splits(n_items, self.heads, self.kv_heads, longest)
            fast_attention.attention_tokens(qkv, self.heads, cache.kv, cache.block_table, step.token_row, step.positions,
                                            step.extra["attn_items"], n_items, splits, self.scale, self.window, out)
        return out


register_mixer("gqa_attention", GroupedQueryAttention)
