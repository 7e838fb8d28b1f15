"""The step function: run a batch of (request, its next tokens) from the cache and return the
logits at the wanted places.

A step runs only the tokens it is given, as one flat batch, whatever mixture of prompt portions
and single decoded tokens it holds.  It is refused as a whole, with nothing applied, when an entry
is malformed or the pages it needs are not there, as the reference refuses a bad plan whole
(helios/crates/helios-hal/src/backends/hopper_sm90/plan_exec.rs:17-41,
helios/crates/helios-hal/src/pool_plan.rs:86-102).
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from .. import ops
from ..cache.manager import NO_PAGE, CacheManager, OutOfPages
from ..csrc import build
from ..models.model import DecoderModel
from .batch import BadStep, MetadataPacker, Row, StepContext, StepEntry


GRAPH_TABLE_STEP = 64  # block-table widths of graphed steps are multiples of this many pages
MAX_GRAPHS = 96


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, use_graphs: bool = True):
        if model.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (no CPU path exists)")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.packer = MetadataPacker(self.device, capacity=1 << 20)  # never reallocated below this: graphs keep its address
        self.planners = model.step_planners()
        build.build_many(model.kernel_modules())
        self.steps_run = 0
        self.use_graphs = use_graphs
        self.graphs: dict = {}
        self._graph_seen: dict = {}
        self._graph_pool = None
        self.graph_launches = 0  # launches of this package's kernels inside replayed graphs

    # ------------------------------------------------------------------ validation
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        if not entries:
            raise BadStep("a step needs at least one entry")
        seen: set[Hashable] = set()
        vocab, limit = self.model.spec.vocab_size, self.model.spec.max_positions
        for entry in entries:
            if entry.request in seen:
                raise BadStep(f"request {entry.request!r} appears twice in one step")
            seen.add(entry.request)
            count = len(entry.tokens)
            if count == 0:
                raise BadStep(f"request {entry.request!r} brings no tokens")
            tokens = np.asarray(entry.tokens)
            if tokens.ndim != 1 or tokens.dtype.kind not in "iu" or int(tokens.min()) < 0 or int(tokens.max()) >= vocab:
                raise BadStep(f"request {entry.request!r}: its tokens must be integers in 0..{vocab - 1}")
            for index in entry.want:
                if isinstance(index, bool) or not isinstance(index, int) or not 0 <= index < count:
                    raise BadStep(f"request {entry.request!r}: wanted index {index!r} is outside its {count} tokens")
            length = self.cache.length(entry.request) if self.cache.has(entry.request) else 0
            if length + count > limit:
                raise BadStep(f"request {entry.request!r} would reach position {length + count}, the model's limit is {limit}")

    # ------------------------------------------------------------------ the batch on the device
    def _context(self, entries: Sequence[StepEntry], extra_arrays=None, pad_tables: bool = False, device_places=None) -> StepContext:
        rows: list[Row] = []
        token_chunks, position_chunks, row_chunks = [], [], []
        want: list[int] = []
        start = 0
        for index, entry in enumerate(entries):
            position, count = self.cache.length(entry.request), len(entry.tokens)
            rows.append(Row(entry.request, start, count, position, self.cache.slot(entry.request)))
            token_chunks.append(np.asarray(entry.tokens, dtype=np.int32))
            position_chunks.append(np.arange(position, position + count, dtype=np.int32))
            row_chunks.append(np.full(count, index, dtype=np.int32))
            want.extend(start + i for i in entry.want)
            start += count
        token_ids, positions, token_row = np.concatenate(token_chunks), np.concatenate(position_chunks), np.concatenate(row_chunks)
        packer = self.packer
        packer.begin()
        packer.add("token_ids", token_ids)
        packer.add("positions", positions)
        packer.add("token_row", token_row)
        packer.add("row_start", [row.start for row in rows] + [int(token_ids.size)])
        packer.add("slots", [row.slot for row in rows])
        if want:
            packer.add("want", want)
        for group in range(len(self.cache.paged)):
            tables = [self.cache.table(group, row.request) for row in rows]
            width = max(1, max(len(t) for t in tables))
            if pad_tables:  # a replayed graph needs the same layout for many steps: widths in steps of GRAPH_TABLE_STEP
                width = -(-width // GRAPH_TABLE_STEP) * GRAPH_TABLE_STEP
            flat: list[int] = []
            for table in tables:
                flat.extend(table)
                flat.extend([NO_PAGE] * (width - len(table)))
            packer.add(f"table{group}", flat, (len(rows), width))
        host = {"positions": positions, "token_row": token_row, "want": want, "page_size": self.cache.page_size}
        if pad_tables:
            host["context_cap"] = width * self.cache.page_size if self.cache.paged else 0
        for key, plan in self.planners.items():
            plan(rows, packer, host)
        for name, (values, shape) in (extra_arrays or {}).items():
            packer.add(name, values, shape)
        if device_places:  # last, so that the other arrays lie where a captured graph expects them
            packer.add("device_token_pairs", [v for index, place in device_places.items() for v in (rows[index].start, place)])
        arrays = packer.finish()
        extra = {k: v for k, v in arrays.items() if k not in ("token_ids", "positions", "token_row", "row_start", "slots", "want")
                 and not k.startswith("table")}
        return StepContext(rows=rows, n_tokens=int(token_ids.size), token_ids=arrays["token_ids"], positions=arrays["positions"],
                           token_row=arrays["token_row"], row_start=arrays["row_start"], want_rows=arrays.get("want"),
                           n_want=len(want), paged_tables=[arrays[f"table{g}"] for g in range(len(self.cache.paged))],
                           slots=arrays["slots"], extra=extra, host=host)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], extra_arrays=None, device_tokens=None) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns float logits [wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``, or None when nothing was wanted.
        ``extra_arrays`` ({name: (int32 values, shape)}) ride along in the step's one host-to-device
        copy and are found in ``self.last_context.extra`` afterwards.
        ``device_tokens`` = (int32 tensor on the device, {index of an entry: index into the tensor}):
        the named entries, of one token each, take that token from the tensor instead of from their
        ``tokens`` (whose value is ignored), so a token sampled by the step before need not pass
        through the host."""
        entries = list(entries)
        self._validate(entries)
        if device_tokens is not None:
            source, places = device_tokens
            if source.dtype != torch.int32 or source.device != self.device or not source.is_contiguous():
                raise BadStep("device tokens must be a contiguous int32 tensor on the engine's device")
            for index, place in places.items():
                if not 0 <= index < len(entries) or len(entries[index].tokens) != 1 or not 0 <= place < source.numel():
                    raise BadStep(f"device token {place} for entry {index}: only a single-token entry can take a token of the tensor")
        added = []
        try:
            for entry in entries:
                if not self.cache.has(entry.request):
                    self.cache.add_request(entry.request)
                    added.append(entry.request)
            self.cache.extend_all([(entry.request, len(entry.tokens)) for entry in entries])
        except OutOfPages:
            for request in added:
                self.cache.free(request)
            raise
        key = self._graph_key(entries, extra_arrays)
        context = self._context(entries, extra_arrays, pad_tables=key is not None,
                                device_places=device_tokens[1] if device_tokens is not None else None)
        self.last_context = context
        if device_tokens is not None and device_tokens[1]:
            ops.place_tokens(context.token_ids, device_tokens[0], context.extra.pop("device_token_pairs"))
        logits = self.model.forward(context, self.cache) if key is None else self._replay(key, context)
        for entry in entries:
            self.cache.advance(entry.request, len(entry.tokens))
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ CUDA graphs for decode steps
    def _graph_key(self, entries: Sequence[StepEntry], extra_arrays):
        """Steps of single decoded tokens whose logits are all wanted repeat with the same shape: their
        launches are captured once per (rows, table width, extra arrays) and replayed, which removes
        the host's launch cost (the reference captures a graph per decode bucket for the same reason:
        helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:510-551)."""
        if not self.use_graphs or any(len(e.tokens) != 1 or list(e.want) != [0] for e in entries):
            return None
        widths = []
        for group in range(len(self.cache.paged)):
            blocks = max(-(-(self.cache.length(e.request) + 1) // self.cache.page_size) for e in entries)
            blocks = max(blocks, max(len(self.cache.table(group, e.request)) for e in entries))
            widths.append(-(-blocks // GRAPH_TABLE_STEP) * GRAPH_TABLE_STEP)
        extras = tuple((name, len(values)) for name, (values, _) in (extra_arrays or {}).items())
        return (len(entries), tuple(widths), extras)

    def _replay(self, key, context: StepContext):
        entry = self.graphs.get(key)
        if entry is None:
            seen = self._graph_seen.get(key, 0) + 1
            self._graph_seen[key] = seen
            if seen < 2 or len(self.graphs) >= MAX_GRAPHS:  # the first step of a shape runs directly (it also warms the libraries up)
                return self.model.forward(context, self.cache)
            from ..ops import native

            before = native.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self.model.forward(context, self.cache)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, logits, native.LAUNCHES[0] - before)
            native.LAUNCHES[0] = before
            self.graphs[key] = entry
        graph, logits, launches = entry
        graph.replay()
        self.graph_launches += launches
        return logits

    def finish(self, request: Hashable) -> None:
        """The request is over: its pages and its state slot go back to the pools."""
        self.cache.free(request)

    def check_device_status(self) -> None:
        ops.raise_on_status(self.device)
