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
from .. import host as host_runtime
from ..cache.manager import CacheManager, OutOfPages
from ..csrc import build
from ..ops import native
from ..models.model import DecoderModel
from .batch import BadStep, MetadataPacker, Rows, StepContext, StepEntry


GRAPH_TABLE_STEP = -64  # block-table widths of graphed steps: 64 pages times a power of two (the runtime's rule for negative steps)
MAX_GRAPHS = 96
GRAPH_MAX_OUTPUT_BYTES = 64 << 20


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, use_graphs: bool = True):
        if model.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only (no CPU path exists)")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.packer = MetadataPacker(self.device, capacity=1 << 20)  # never reallocated below this: graphs keep its address
        self._packer_generation = self.packer.generation
        self.planners = model.step_planners()
        build.build_many(model.kernel_modules())
        self.steps_run = 0
        self.use_graphs = use_graphs
        self.graphs: dict = {}
        self._graph_seen: dict = {}
        self._graph_pool = None
        self.graph_launches = 0  # launches of this package's kernels inside replayed graphs

    # ------------------------------------------------------------------ validation
    def _validate(self, entries: Sequence[StepEntry]) -> list[np.ndarray]:
        """Refuses a malformed step; returns every entry's tokens as an array."""
        if not entries:
            raise BadStep("a step needs at least one entry")
        arrays: list[np.ndarray] = []
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
            arrays.append(tokens)
            for index in entry.want:
                if isinstance(index, bool) or not isinstance(index, int) or not 0 <= index < count:
                    raise BadStep(f"request {entry.request!r}: wanted index {index!r} is outside its {count} tokens")
            length = self.cache.length(entry.request) if self.cache.has(entry.request) else 0
            if length + count > limit:
                raise BadStep(f"request {entry.request!r} would reach position {length + count}, the model's limit is {limit}")
        return arrays

    # ------------------------------------------------------------------ the batch on the device
    def _context(self, names, keys: np.ndarray, counts: np.ndarray, tokens: np.ndarray, want: np.ndarray, extra_arrays=None,
                 pad_tables: bool = False, device_places=None) -> StepContext:
        packer = self.packer
        packer.begin()
        # a replayed graph needs the same layout for many steps: its table widths are 64 pages times a power of two
        packer.add_step(self.cache, keys, counts, tokens, want, GRAPH_TABLE_STEP if pad_tables else 0)
        starts = packer.view("row_start")
        starts = starts[:-1].copy()
        rows = Rows(names, starts, counts, packer.view("positions")[starts], packer.view("slots").copy())
        host = {"page_size": self.cache.page_size}
        if pad_tables:
            widest = max((packer.view(f"table{g}").shape[1] for g in range(len(self.cache.paged))), default=0)
            host["context_cap"] = widest * self.cache.page_size
        for key, plan in self.planners.items():
            plan(rows, packer, host)
        for name, (values, shape) in (extra_arrays or {}).items():
            packer.add(name, values, shape)
        if device_places:  # last, so that the other arrays lie where a captured graph expects them
            packer.add("device_token_pairs", [v for index, place in device_places.items() for v in (int(starts[index]), place)])
        arrays = packer.finish()
        if packer.generation != self._packer_generation:  # the device buffer moved: captured graphs point at the old one
            self.graphs.clear()
            self._packer_generation = packer.generation
        extra = {k: v for k, v in arrays.items() if k not in ("token_ids", "positions", "token_row", "row_start", "slots", "want")
                 and not k.startswith("table")}
        return StepContext(rows=rows, n_tokens=len(tokens), token_ids=arrays["token_ids"], positions=arrays["positions"],
                           token_row=arrays["token_row"], row_start=arrays["row_start"], want_rows=arrays.get("want"),
                           n_want=len(want), paged_tables=[arrays[f"table{g}"] for g in range(len(self.cache.paged))],
                           slots=arrays["slots"], extra=extra, host=host)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry], extra_arrays=None, device_tokens=None) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns float logits [wanted, vocab] on the device, in the
        order of the entries and of each entry's ``want``, or None when nothing was wanted.  The tensor
        may be written again by the next step (a replayed graph writes its output in place): copy it to keep it.
        ``extra_arrays`` ({name: (int32 values, shape)}) ride along in the step's one host-to-device
        copy and are found in ``self.last_context.extra`` afterwards.
        ``device_tokens`` = (int32 tensor on the device, {index of an entry: index into the tensor}):
        the named entries, of one token each, take that token from the tensor instead of from their
        ``tokens`` (whose value is ignored), so a token sampled by the step before need not pass
        through the host."""
        entries = list(entries)
        token_arrays = self._validate(entries)
        self._check_device_tokens(device_tokens, [len(e.tokens) for e in entries])
        added = []
        try:
            for entry in entries:
                if not self.cache.has(entry.request):
                    self.cache.add_request(entry.request)
                    added.append(entry.request)
            keys = np.asarray([self.cache.keys.known(entry.request) for entry in entries], dtype=np.int64)
            counts = np.asarray([len(entry.tokens) for entry in entries], dtype=np.int32)
            self.cache.extend_keys(keys, counts)
        except OutOfPages:
            for request in added:
                self.cache.free(request)
            raise
        tokens = np.concatenate(token_arrays).astype(np.int32, copy=False)
        starts = np.concatenate(([0], np.cumsum(counts)[:-1]))
        want = np.asarray([int(starts[i]) + w for i, entry in enumerate(entries) for w in entry.want], dtype=np.int32)
        return self._run([entry.request for entry in entries], keys, counts, tokens, want, extra_arrays, device_tokens)

    def step_arrays(self, names, keys: np.ndarray, counts: np.ndarray, tokens: np.ndarray, want: np.ndarray, extra_arrays=None,
                    device_tokens=None) -> Optional[torch.Tensor]:
        """:meth:`step` for callers that hold the batch as arrays already (the generation loop): ``keys`` are the cache
        manager's keys of live requests (int64), ``counts`` the tokens per row, ``tokens`` all rows' tokens back to back,
        ``want`` flat indices among them (all int32).  The same checks, done on whole arrays."""
        vocab, limit = self.model.spec.vocab_size, self.model.spec.max_positions
        if len(keys) == 0 or len(counts) != len(keys) or int(counts.sum()) != len(tokens):
            raise BadStep("a step needs at least one row, and as many tokens as its rows count")
        if len(np.unique(keys)) != len(keys):
            raise BadStep("a request appears twice in one step")
        if int(counts.min()) < 1:
            raise BadStep("a row brings no tokens")
        if int(tokens.min()) < 0 or int(tokens.max()) >= vocab:
            raise BadStep(f"tokens must be integers in 0..{vocab - 1}")
        if len(want) and (int(want.min()) < 0 or int(want.max()) >= len(tokens)):
            raise BadStep("a wanted place is outside the step's tokens")
        lengths, slots = np.empty(len(keys), np.int32), np.empty(len(keys), np.int32)
        host_runtime.check(host_runtime.library().hb_cache_lengths(self.cache.native, len(keys), host_runtime.address(keys), host_runtime.address(lengths),
                                                                   host_runtime.address(slots)))
        if int(lengths.min()) < 0:
            raise BadStep("a row names a request the cache does not know")
        if int((lengths + counts).max()) > limit:
            raise BadStep(f"a request would pass the model's limit of {limit} positions")
        self._check_device_tokens(device_tokens, counts)
        self.cache.extend_keys(keys, counts)
        return self._run(names, keys, counts, tokens, want, extra_arrays, device_tokens)

    def _check_device_tokens(self, device_tokens, counts) -> None:
        if device_tokens is None:
            return
        source, places = device_tokens
        if source.dtype != torch.int32 or source.device != self.device or not source.is_contiguous():
            raise BadStep("device tokens must be a contiguous int32 tensor on the engine's device")
        for index, place in places.items():
            if not 0 <= index < len(counts) or counts[index] != 1 or not 0 <= place < source.numel():
                raise BadStep(f"device token {place} for entry {index}: only a single-token entry can take a token of the tensor")

    def _run(self, names, keys, counts, tokens, want, extra_arrays, device_tokens) -> Optional[torch.Tensor]:
        key = self._graph_key(keys, counts, want, extra_arrays)
        context = self._context(names, keys, counts, tokens, want, extra_arrays, pad_tables=key is not None,
                                device_places=device_tokens[1] if device_tokens is not None else None)
        self.last_context = context
        if device_tokens is not None and device_tokens[1]:
            ops.place_tokens(context.token_ids, device_tokens[0], context.extra.pop("device_token_pairs"))
        with native.stream_bound():
            logits = self.model.forward(context, self.cache) if key is None else self._replay(key, context)
        self.cache.advance_keys(keys, counts)
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------------ CUDA graphs for steps whose shape repeats
    def _graph_key(self, keys: np.ndarray, counts: np.ndarray, want: np.ndarray, extra_arrays):
        """Steps of the same shape (tokens per row, number of wanted places, block-table widths rounded up to 64 pages
        times a power of two, extra arrays) launch the same kernels with the same arguments: everything that
        differs between them lies in the metadata buffer.  Such a step is captured into a CUDA graph when its
        shape comes again and replayed from then on, which removes the host's launch cost (the reference captures
        a graph per decode bucket and per prefill capacity for the same reason:
        helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:510-551).  Steps of single decoded tokens
        are captured at their second sighting, other shapes at their third."""
        if not self.use_graphs:
            return None
        decode = len(want) == len(counts) and int(counts.max()) == 1 and np.array_equal(want, np.arange(len(counts)))
        if not decode and len(want) * self.model.spec.vocab_size * 4 > GRAPH_MAX_OUTPUT_BYTES:
            return None  # a graph keeps its output alive: not for steps that want logits at hundreds of places
        widths = np.zeros(max(1, len(self.cache.paged)), dtype=np.int32)
        host_runtime.check(host_runtime.library().hb_step_decode_widths(self.cache.native, len(keys), host_runtime.address(keys), GRAPH_TABLE_STEP,
                                                                        host_runtime.address(widths)))
        extras = tuple((name, len(values)) for name, (values, _) in (extra_arrays or {}).items())
        shape = len(keys) if decode else tuple(counts.tolist())
        return (shape, len(want), tuple(widths[: len(self.cache.paged)].tolist()), extras)

    def _replay(self, key, context: StepContext):
        entry = self.graphs.get(key)
        if entry is None:
            if len(self._graph_seen) > 4 * MAX_GRAPHS:  # shapes that never came again are forgotten
                self._graph_seen.clear()
            seen = self._graph_seen.get(key, 0) + 1
            self._graph_seen[key] = seen
            needed = 2 if isinstance(key[0], int) else 3
            if seen < needed:  # the first steps of a shape run directly (they also warm the libraries up)
                return self.model.forward(context, self.cache)
            if len(self.graphs) >= MAX_GRAPHS:  # the shape that was replayed longest ago makes room
                self.graphs.pop(next(iter(self.graphs)))
            before = native.LAUNCHES[0]
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=self._graph_pool), native.stream_bound():
                logits = self.model.forward(context, self.cache)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, logits, native.LAUNCHES[0] - before)
            native.LAUNCHES[0] = before
            self.graphs[key] = entry
        self.graphs[key] = self.graphs.pop(key)  # most recently used last
        graph, logits, launches = entry
        graph.replay()
        self.graph_launches += launches
        return logits

    def finish(self, request: Hashable) -> None:
        """The request is over: its pages and its state slot go back to the pools."""
        self.cache.free(request)

    def check_device_status(self) -> None:
        ops.raise_on_status(self.device)
