"""A decoder built from a :class:`ModelSpec`: embedding, the scheduled layers, final norm, head.

The model knows nothing about any architecture; it instantiates the registered parts the spec
names, collects the tensor names and shapes they want, hands loaded tensors back to them, and runs
the schedule over the tokens of one step.  The order of operations follows the reference's forward
pass (helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:646-811): embedding, per layer
norm -> mixer -> residual+norm -> feed-forward, then the final norm and the head on the rows whose
logits are wanted only (session.rs:826-831).
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..engine.batch import PagedView, StateView, StepContext
from ..parts import base as parts
from ..parts.base import BuildContext, PagedTokens, RequestState, WeightSpec
from ..parts.spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = device
        self.build = BuildContext(dtype=dtype, device=device, max_positions=spec.max_positions, shared={})
        self.embedding = parts.make(parts.EMBEDDINGS, spec.embedding, self.build)
        self.layers = []
        for layer in spec.layers:
            mixer = parts.make(parts.MIXERS, layer.mixer, self.build)
            feed_forward = parts.make(parts.FEED_FORWARDS, layer.feed_forward, self.build)
            norms = {name: parts.make(parts.NORMS, norm, self.build) for name, norm in layer.norms.items()}
            if layer.arrangement not in parts.ARRANGEMENTS:
                raise KeyError(f"no arrangement {layer.arrangement!r} is registered")
            self.layers.append(parts.ARRANGEMENTS[layer.arrangement](mixer, feed_forward, norms))
        self.final_norm = parts.make(parts.NORMS, spec.final_norm, self.build)
        self.head = parts.make(parts.HEADS, spec.head, self.build)
        for index, run in enumerate(spec.schedule):
            owns = self.layers[run.layer].mixer.cache_request() is not None
            if run.reads_cache_of is None and not owns and getattr(self.layers[run.layer].mixer, "shares_kv", False):
                raise ValueError(f"schedule[{index}]: the mixer reads a shared cache but the entry names none")

    # ------------------------------------------------------------------ tensors
    def _named_parts(self):
        yield self.spec.embedding.prefix, self.embedding
        for layer_spec, layer in zip(self.spec.layers, self.layers):
            yield layer_spec.mixer.prefix, layer.mixer
            yield layer_spec.feed_forward.prefix, layer.feed_forward
            for name, norm_spec in layer_spec.norms.items():
                yield norm_spec.prefix, layer.norms[name]
        yield self.spec.final_norm.prefix, self.final_norm
        yield self.spec.head.prefix, self.head

    def expected_tensors(self) -> dict[str, WeightSpec]:
        expected: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for name, wanted in part.weights().items():
                expected[prefix + name] = wanted
        return expected

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """``tensors`` by full name, on the device, already checked against ``expected_tensors``."""
        for prefix, part in self._named_parts():
            part.load({name: tensors[prefix + name] for name in part.weights()})
        if self.head.wants_shared_table():
            table = self.embedding.shared_table()
            if table is None:
                raise ValueError("the head is tied to the embedding, which has no table to share")
            self.head.use_shared_table(table)

    def cache_users(self) -> list[tuple[int, PagedTokens | RequestState]]:
        """(schedule entry, what its mixer keeps) for every entry that owns a cache."""
        users = []
        for index, run in enumerate(self.spec.schedule):
            if run.reads_cache_of is not None:
                continue
            need = self.layers[run.layer].mixer.cache_request()
            if need is not None:
                users.append((index, need))
        return users

    def kernel_modules(self) -> list[tuple[str, dict]]:
        modules: list[tuple[str, dict]] = []
        for _, part in self._named_parts():
            modules += part.kernel_modules()
        return modules

    def step_planners(self) -> dict:
        """Per-step metadata some parts need beyond the common arrays: ``{key: plan(rows, packer)}``,
        merged over all parts so that parts with the same needs share one plan."""
        planners: dict = {}
        for _, part in self._named_parts():
            planners.update(getattr(part, "step_plans", lambda: {})())
        return planners

    # ------------------------------------------------------------------ one step
    def forward(self, step: StepContext, cache) -> Optional[torch.Tensor]:
        """Run the tokens of ``step`` from and into ``cache``; float logits [wanted, vocab] or None."""
        h = self.embedding.forward(step.token_ids)
        delta = None
        for index, run in enumerate(self.spec.schedule):
            owner = index if run.reads_cache_of is None else run.reads_cache_of
            view = self._cache_view(owner, step, cache)
            h, delta = self.layers[run.layer].forward(h, delta, step, view, run.reads_cache_of is None)
        if step.n_want == 0:
            # the last pending add is never read: keys and values are already in the cache
            return None
        x = self.final_norm.forward(h, delta, step.want_rows)
        return self.head.forward(x)

    def _cache_view(self, entry: int, step: StepContext, cache):
        if cache is None or not cache.has_user(entry):
            return None
        kind, group, _ = cache.where(entry)
        if kind == "paged":
            return PagedView(cache.paged_storage(entry), step.paged_tables[group], cache.page_size, group)
        return StateView(cache.state_storage(entry), step.slots, [int(slot) for slot in step.rows.slots])
