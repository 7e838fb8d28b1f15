"""The parts alone against their plain formulas, and the generality of the composition: a model with
different mixers in different layers, a layer that runs twice, a layer that reads another layer's
cache, a windowed cache group; and a toy mixer with state of its own that is defined here, registered
and stepped without touching the package."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def build_context(dtype, max_positions=512):
    from hyperion_b200.parts import BuildContext

    return BuildContext(dtype=dtype, device=DEV, max_positions=max_positions, shared={})


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2 ** -7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from hyperion_b200.parts import NORMS, PartSpec, base

    part = base.make(NORMS, PartSpec("rmsnorm", "n.", {"hidden_size": 200, "eps": 1e-5}), build_context(dtype))
    assert part.weights()["weight"].shape == (200,)
    w = (1 + rnd(200, seed=1, scale=0.1)).to(torch.bfloat16)
    part.load({"weight": w.to(DEV)})
    h, delta = rnd(5, 200, seed=2), rnd(5, 200, seed=3).to(dtype)
    hd = h.to(DEV)
    out = part.forward(hd, delta.to(DEV))
    want = plain.rmsnorm(h.double() + delta.double(), w.double(), 1e-5)
    assert (out.cpu().double() - want).abs().max() <= tol(dtype) * want.abs().max()
    assert torch.allclose(hd.cpu(), h + delta.float(), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(dtype):
    from hyperion_b200.parts import FEED_FORWARDS, PartSpec, base

    part = base.make(FEED_FORWARDS, PartSpec("swiglu", "m.", {"hidden_size": 96, "intermediate_size": 200}), build_context(dtype))
    names = part.weights()
    assert names["gate_proj.weight"].shape == (200, 96) and names["down_proj.weight"].shape == (96, 200)
    tensors = {n: rnd(*s.shape, seed=i, scale=0.1).to(torch.bfloat16) for i, (n, s) in enumerate(names.items())}
    part.load({n: (t.float() if dtype == torch.float32 else t).to(DEV) for n, t in tensors.items()})
    x = rnd(7, 96, seed=9).to(dtype)
    out = part.forward(x.to(DEV), None)
    want = plain.swiglu_mlp(x.double(), *(tensors[n].double() for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    assert (out.cpu().double() - want).abs().max() <= tol(dtype) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_position_part(dtype):
    from hyperion_b200.parts import POSITIONS, PartSpec, base

    part = base.make(POSITIONS, PartSpec("rope", "", {"head_dim": 24, "base": 5e5, "max_positions": 300}), build_context(dtype))
    x = rnd(4, 3 * 24 + 10, seed=4).to(dtype)
    positions = torch.tensor([0, 7, 150, 299], dtype=torch.int32)
    xd = x.to(DEV).clone()
    part.apply_(xd, 3, 24, positions.to(DEV))
    cos, sin = plain.rope_tables(positions, 24, 5e5)
    want = plain.rope(x.double()[:, :72].view(4, 3, 24), cos, sin).reshape(4, 72)
    assert (xd.cpu().double()[:, :72] - want).abs().max() <= tol(dtype) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from hyperion_b200.parts import EMBEDDINGS, HEADS, PartSpec, base

    sizes = {"vocab_size": 301, "hidden_size": 40}
    embedding = base.make(EMBEDDINGS, PartSpec("token_embedding", "e.", sizes), build_context(dtype))
    head = base.make(HEADS, PartSpec("linear_head", "h.", {**sizes, "tied": True}), build_context(dtype))
    assert head.weights() == {}
    table = rnd(301, 40, seed=5).to(torch.bfloat16)
    embedding.load({"weight": (table.float() if dtype == torch.float32 else table).to(DEV)})
    assert head.wants_shared_table()
    head.use_shared_table(embedding.shared_table())
    ids = torch.tensor([300, 0, 17], dtype=torch.int32)
    h = embedding.forward(ids.to(DEV))
    assert torch.equal(h.cpu(), table.float()[ids.long()])
    x = rnd(3, 40, seed=6).to(dtype)
    logits = head.forward(x.to(DEV))
    assert logits.dtype == torch.float32
    want = x.double() @ table.double().t()
    assert (logits.cpu().double() - want).abs().max() <= tol(dtype) * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """The attention part with a cache of its own: a prompt portion, then two more steps."""
    from hyperion_b200.cache import CacheManager
    from hyperion_b200.engine.batch import PagedView
    from hyperion_b200.parts import MIXERS, PartSpec, base

    hidden, heads, kv_heads, d = 80, 6, 3, 16
    spec = PartSpec("gqa_attention", "a.", {"hidden_size": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": d, "bias": True,
                                            "position": PartSpec("rope", "", {"head_dim": d, "base": 1e4, "max_positions": 128})})
    part = base.make(MIXERS, spec, build_context(dtype, 128))
    tensors = {n: rnd(*s.shape, seed=20 + i, scale=0.15).to(torch.bfloat16) for i, (n, s) in enumerate(part.weights().items())}
    part.load({n: (t.float() if dtype == torch.float32 else t).to(DEV) for n, t in tensors.items()})
    cache = CacheManager([(0, part.cache_request())], page_size=8, num_pages=6, max_requests=2, dtype=dtype, device=DEV)
    cache.add_request("r")
    x = rnd(21, hidden, seed=30).to(dtype)
    w = {"a." + n: t for n, t in tensors.items()}
    dims = {"heads": heads, "kv_heads": kv_heads, "head_dim": d, "theta": 1e4}
    want = plain.attention_block(x.double(), {k: v.double() for k, v in w.items()}, "a.", dims, torch.arange(21))

    @dataclass
    class Step:
        n_tokens: int
        positions: torch.Tensor
        token_row: torch.Tensor
        rows: list
        host: dict
        extra: dict

    from hyperion_b200.engine.batch import MetadataPacker, Row

    at = 0
    for count in (17, 1, 3):
        cache.extend("r", count)
        rows = [Row("r", 0, count, at, cache.slot("r"))]
        packer = MetadataPacker(DEV)
        packer.begin()
        host: dict = {}
        for plan in part.step_plans().values():
            plan(rows, packer, host)
        extra = packer.finish()
        step = Step(count, torch.arange(at, at + count, dtype=torch.int32, device=DEV), torch.zeros(count, dtype=torch.int32, device=DEV),
                    rows, host, extra)
        table = torch.tensor([cache.table(0, "r")], dtype=torch.int32, device=DEV)
        out = part.forward(x[at:at + count].to(DEV), step, PagedView(cache.paged_storage(0), table, 8, 0), True)
        assert (out.cpu().double() - want[at:at + count]).abs().max() <= 2 * tol(dtype) * want.abs().max()
        cache.advance("r", count)
        at += count


# ------------------------------------------------------------------------------------------------
# A model whose layers differ: full attention, windowed attention run twice, and a layer that reads
# the first layer's cache.  Its architecture is registered here, not in the package.
MIXED = {"architectures": ["TestMixedLM"], "hidden": 96, "vocab": 211, "inter": 136, "eps": 1e-5, "window": 24, "max_positions": 256}


def mixed_spec(c):
    from hyperion_b200.parts import LayerSpec, ModelSpec, PartSpec, Run

    rope = PartSpec("rope", "", {"head_dim": 16, "base": 1e4, "max_positions": c["max_positions"]})

    def attention(prefix, kv_heads, **more):
        return PartSpec("gqa_attention", prefix, {"hidden_size": c["hidden"], "heads": 6, "kv_heads": kv_heads, "head_dim": 16,
                                                   "bias": True, "position": rope, **more})

    def layer(i, mixer):
        p = f"layers.{i}."
        norm = {"hidden_size": c["hidden"], "eps": c["eps"]}
        return LayerSpec("prenorm", mixer, PartSpec("swiglu", p + "mlp.", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]}),
                         {"input": PartSpec("rmsnorm", p + "n1.", norm), "post_mixer": PartSpec("rmsnorm", p + "n2.", norm)})

    layers = (layer(0, attention("layers.0.attn.", 2)), layer(1, attention("layers.1.attn.", 3, window=c["window"])),
              layer(2, attention("layers.2.attn.", 2, shares_kv=True)))
    sizes = {"vocab_size": c["vocab"], "hidden_size": c["hidden"]}
    return ModelSpec("TestMixedLM", c["hidden"], c["vocab"], c["max_positions"], PartSpec("token_embedding", "embed.", sizes), layers,
                     (Run(0), Run(1), Run(1), Run(2, reads_cache_of=0)), PartSpec("rmsnorm", "norm.", {"hidden_size": c["hidden"], "eps": c["eps"]}),
                     PartSpec("linear_head", "head.", {**sizes, "tied": False}))


def mixed_plain(c, w, ids):
    """The same model with the plain functions, whole sequence."""
    w = {k: v.double() for k, v in w.items()}
    t = len(ids)
    positions = torch.arange(t)
    cos, sin = plain.rope_tables(positions, 16, 1e4)
    h = plain.embedding(w["embed.weight"], torch.tensor(ids))
    kept = {}

    def attend(layer, x, kv_heads, window=None, shared=None):
        p = f"layers.{layer}.attn."
        q = plain.rope(plain.linear(x, w[p + "q_proj.weight"], w[p + "q_proj.bias"]).view(t, 6, 16), cos, sin)
        if shared is None:
            k = plain.rope(plain.linear(x, w[p + "k_proj.weight"], w[p + "k_proj.bias"]).view(t, kv_heads, 16), cos, sin)
            v = plain.linear(x, w[p + "v_proj.weight"], w[p + "v_proj.bias"]).view(t, kv_heads, 16)
            kept[layer] = (k, v)
        else:
            k, v = kept[shared]
        a = plain.attention(q, k, v, positions, positions, 0.25, window)
        return plain.linear(a.reshape(t, -1), w[p + "o_proj.weight"])

    for layer, kv_heads, window, shared in ((0, 2, None, None), (1, 3, c["window"], None), (1, 3, c["window"], None), (2, 2, None, 0)):
        p = f"layers.{layer}."
        h = h + attend(layer, plain.rmsnorm(h, w[p + "n1.weight"], c["eps"]), kv_heads, window, shared)
        x = plain.rmsnorm(h, w[p + "n2.weight"], c["eps"])
        h = h + plain.swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], c["eps"]), w["head.weight"])


@pytest.fixture(scope="module")
def mixed_folder(tmp_path_factory):
    from hyperion_b200.models import Architecture, register_architecture
    from hyperion_b200.weights import write_model_folder

    register_architecture(Architecture("TestMixedLM", lambda document: dict(document), mixed_spec, lambda config: dict(config)))
    return write_model_folder(tmp_path_factory.mktemp("mixed") / "m", "TestMixedLM", MIXED, seed=4, std=0.08)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_different_kinds_twice_run_and_shared_cache(mixed_folder, dtype):
    from hyperion_b200.api import Engine
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.weights import read_all

    weights = read_all(mixed_folder)
    assert "layers.2.attn.k_proj.weight" not in weights and "layers.1.attn.k_proj.bias" in weights
    g = torch.Generator().manual_seed(0)
    requests = {name: torch.randint(0, MIXED["vocab"], (n,), generator=g).tolist() for name, n in (("a", 120), ("b", 75), ("c", 140))}
    want = {name: mixed_plain(MIXED, weights, ids).numpy() for name, ids in requests.items()}
    engine = Engine.from_folder(mixed_folder, dtype=dtype, page_size=8, max_tokens=232, max_requests=3)
    cache = engine.cache
    assert len(cache.paged) == 2 and cache.paged[0].users == [0] and cache.paged[1].users == [1, 2]  # entry 3 owns no cache
    tolerance = 2e-5 if dtype == "float32" else 2.5e-2
    fed = {name: 0 for name in requests}
    sizes = [9, 2, 30, 1, 5, 17, 1, 1, 40, 3]
    k = 0
    order = ["a", "b"]
    cut = {name: [] for name in requests}  # the logits of this cutting, per request in position order
    while order:
        entries = []
        for name in list(order):
            n = min(sizes[k % len(sizes)], len(requests[name]) - fed[name])
            k += 1
            entries.append(StepEntry(name, requests[name][fed[name]:fed[name] + n], list(range(n))))
        logits = engine.step(entries).cpu().numpy()
        row = 0
        for entry in entries:
            n = len(entry.tokens)
            ref = want[entry.request][fed[entry.request]:fed[entry.request] + n]
            assert np.abs(logits[row:row + n] - ref).max() <= tolerance * np.abs(ref).max(), (entry.request, fed[entry.request])
            cut[entry.request].append(logits[row:row + n].copy())
            row += n
            fed[entry.request] += n
            if fed[entry.request] == len(requests[entry.request]):
                engine.finish(entry.request)
                order.remove(entry.request)
                if entry.request == "b":
                    order.append("c")  # takes over the pages b and the windows gave back
        cache.check()
    engine.check()
    # the windowed group held far fewer pages than the full one at the end of a long request
    assert cache.free_pages(1) == cache.num_pages
    if dtype == "float32":  # each request whole in one step gives the very bits of the cutting above: window, shared cache and all
        for name, ids in requests.items():
            whole = engine.step([StepEntry(("whole", name), ids, list(range(len(ids))))]).cpu().numpy()
            engine.finish(("whole", name))
            assert np.array_equal(whole.view(np.uint32), np.concatenate(cut[name]).view(np.uint32)), name


# ------------------------------------------------------------------------------------------------
# A toy mixer with state of its own: an exponential moving sum per request, kept in a state slot.
TOY = {"architectures": ["TestToyStateLM"], "hidden": 48, "vocab": 97, "inter": 64, "eps": 1e-6, "decay": 0.9, "max_positions": 128}


def register_toy():
    from hyperion_b200.models import Architecture, register_architecture
    from hyperion_b200.parts import LayerSpec, Mixer, ModelSpec, PartSpec, RequestState, Run, WeightSpec, register_mixer

    class MovingSum(Mixer):
        """y_t = (s_t) W_out with s_t = decay * s_{t-1} + x_t W_in; s lives in the request's state slot."""

        def __init__(self, spec, build):
            super().__init__(spec, build)
            self.hidden, self.decay = spec.params["hidden_size"], spec.params["decay"]

        def weights(self):
            return {"in.weight": WeightSpec((self.hidden, self.hidden)), "out.weight": WeightSpec((self.hidden, self.hidden))}

        def load(self, tensors):
            self.w_in, self.w_out = tensors["in.weight"].float(), tensors["out.weight"].float()

        def cache_request(self):
            return RequestState((self.hidden,), torch.float32)

        def forward(self, x, step, cache, own_cache):
            u = x.float() @ self.w_in.t()
            out = torch.empty_like(u)
            for row in step.rows:
                s = cache.state[row.slot]
                for t in range(row.start, row.start + row.count):
                    s = self.decay * s + u[t]
                    out[t] = s
                cache.state[row.slot] = s
            return (out @ self.w_out.t()).to(self.dtype)

    def spec(c):
        sizes = {"vocab_size": c["vocab"], "hidden_size": c["hidden"]}
        norm = {"hidden_size": c["hidden"], "eps": c["eps"]}
        layers = tuple(LayerSpec("prenorm", PartSpec("test_moving_sum", f"l{i}.mix.", {"hidden_size": c["hidden"], "decay": c["decay"]}),
                                 PartSpec("swiglu", f"l{i}.mlp.", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]}),
                                 {"input": PartSpec("rmsnorm", f"l{i}.n1.", norm), "post_mixer": PartSpec("rmsnorm", f"l{i}.n2.", norm)})
                       for i in range(2))
        return ModelSpec("TestToyStateLM", c["hidden"], c["vocab"], c["max_positions"], PartSpec("token_embedding", "embed.", sizes), layers,
                         (Run(0), Run(1)), PartSpec("rmsnorm", "norm.", norm), PartSpec("linear_head", "head.", {**sizes, "tied": True}))

    register_mixer("test_moving_sum", MovingSum)
    register_architecture(Architecture("TestToyStateLM", lambda document: dict(document), spec, lambda config: dict(config)))


def toy_plain(c, w, ids):
    w = {k: v.double() for k, v in w.items()}
    h = plain.embedding(w["embed.weight"], torch.tensor(ids))
    for i in range(2):
        x = plain.rmsnorm(h, w[f"l{i}.n1.weight"], c["eps"])
        u = x @ w[f"l{i}.mix.in.weight"].t()
        s = torch.zeros(c["hidden"], dtype=torch.float64)
        states = []
        for t in range(len(ids)):
            s = c["decay"] * s + u[t]
            states.append(s)
        h = h + torch.stack(states) @ w[f"l{i}.mix.out.weight"].t()
        x = plain.rmsnorm(h, w[f"l{i}.n2.weight"], c["eps"])
        h = h + plain.swiglu_mlp(x, w[f"l{i}.mlp.gate_proj.weight"], w[f"l{i}.mlp.up_proj.weight"], w[f"l{i}.mlp.down_proj.weight"])
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], c["eps"]), w["embed.weight"])


def test_a_toy_mixer_with_its_own_state_registers_builds_and_steps(tmp_path):
    from hyperion_b200.api import Engine
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.weights import read_all, write_model_folder

    register_toy()
    folder = write_model_folder(tmp_path / "toy", "TestToyStateLM", TOY, seed=8, std=0.1)
    weights = read_all(folder)
    engine = Engine.from_folder(folder, dtype="float32", page_size=16, max_tokens=64, max_requests=2)
    assert not engine.cache.paged and [s.users for s in engine.cache.states][0] == [0, 1]
    g = torch.Generator().manual_seed(1)
    a, b, c = (torch.randint(0, TOY["vocab"], (n,), generator=g).tolist() for n in (30, 22, 18))
    want = {"a": toy_plain(TOY, weights, a).numpy(), "b": toy_plain(TOY, weights, b).numpy(), "c": toy_plain(TOY, weights, c).numpy()}
    got_a = [engine.step([StepEntry("a", a[:11], list(range(11)))]).cpu().numpy()]
    mixed = engine.step([StepEntry("a", a[11:12], [0]), StepEntry("b", b, list(range(22)))]).cpu().numpy()
    got_a.append(mixed[:1])
    assert np.abs(mixed[1:] - want["b"]).max() <= 1e-4 * np.abs(want["b"]).max()
    engine.finish("b")
    # c takes b's slot: its state must start from zero, not from what b left
    mixed = engine.step([StepEntry("c", c, list(range(18))), StepEntry("a", a[12:], list(range(18)))]).cpu().numpy()
    assert engine.cache.slot("c") == 1
    got_a.append(mixed[18:])
    assert np.abs(mixed[:18] - want["c"]).max() <= 1e-4 * np.abs(want["c"]).max()
    assert np.abs(np.concatenate(got_a) - want["a"]).max() <= 1e-4 * np.abs(want["a"]).max()
    engine.finish("a")
    engine.finish("c")
    # generation: the model keeps no pages, so admission asks for none (the cache of 64 tokens would not hold these requests
    # if they were counted in pages) and only the two request slots bound how many run at a time
    from hyperion_b200.sampling import SamplingParams

    prompts = [a, b, c]
    engine.runner.use_graphs = False  # this toy decides on the host by slot numbers, which a replayed graph would repeat
    tokens, reasons = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=60, ignore_eos=True), return_reasons=True, lookahead=False)
    assert reasons == ["length"] * 3 and [len(t) for t in tokens] == [60, 60, 60]
    for prompt, made in zip(prompts, tokens):
        ref = toy_plain(TOY, weights, prompt + made).numpy()
        for i, token in enumerate(made[:8]):
            row = ref[len(prompt) + i - 1]
            assert row.max() - row[token] <= 1e-4 * np.abs(row).max()


# ------------------------------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, both defined here.
ROUTED = {"architectures": ["TestRoutedLM"], "hidden": 64, "vocab": 131, "inter": 96, "experts": 4, "expert_inter": 40, "eps": 1e-6,
          "max_positions": 128}


def register_routed():
    from hyperion_b200.models import Architecture, register_architecture
    from hyperion_b200.parts import (FeedForward, LayerSpec, ModelSpec, PartSpec, PositionEncoding, Run, WeightSpec, register_feed_forward,
                                     register_position)

    class TopOneExperts(FeedForward):
        """Router logits in float; every token goes to its best expert (a small GELU MLP); output scaled by the router's softmax weight."""

        def __init__(self, spec, build):
            super().__init__(spec, build)
            p = spec.params
            self.hidden, self.experts, self.inter = p["hidden_size"], p["experts"], p["expert_inter"]

        def weights(self):
            return {"router.weight": WeightSpec((self.experts, self.hidden)), "w1": WeightSpec((self.experts, self.inter, self.hidden)),
                    "w2": WeightSpec((self.experts, self.hidden, self.inter))}

        def load(self, tensors):
            self.router, self.w1, self.w2 = (tensors[n].float() for n in ("router.weight", "w1", "w2"))

        def forward(self, x, step):
            xf = x.float()
            probs = torch.softmax(xf @ self.router.t(), dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros_like(xf)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    hidden = torch.nn.functional.gelu(xf[rows] @ self.w1[e].t())
                    out[rows] = (hidden @ self.w2[e].t()) * weight[rows, None]
            return out.to(self.dtype)

    class InterleavedRotary(PositionEncoding):
        """Rotates the pairs (2i, 2i+1) of every head by position * base^(-2i/d): another convention than rotate-half."""

        def __init__(self, spec, build):
            super().__init__(spec, build)
            d, base = spec.params["head_dim"], spec.params["base"]
            inv = base ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
            angle = torch.arange(build.max_positions, dtype=torch.float64)[:, None] * inv[None]
            self.cos, self.sin = angle.cos().float().to(build.device), angle.sin().float().to(build.device)

        def apply_(self, x, heads, head_dim, positions):
            t = x.shape[0]
            view = x[:, : heads * head_dim].float().reshape(t, heads, head_dim // 2, 2)
            c, s = self.cos[positions.long()][:, None, :], self.sin[positions.long()][:, None, :]
            even, odd = view[..., 0] * c - view[..., 1] * s, view[..., 1] * c + view[..., 0] * s
            x[:, : heads * head_dim] = torch.stack([even, odd], dim=-1).reshape(t, heads * head_dim).to(x.dtype)

    def spec(c):
        sizes = {"vocab_size": c["vocab"], "hidden_size": c["hidden"]}
        norm = {"hidden_size": c["hidden"], "eps": c["eps"]}

        def attention(i, position):
            return PartSpec("gqa_attention", f"l{i}.attn.", {"hidden_size": c["hidden"], "heads": 4, "kv_heads": 2, "head_dim": 16, "bias": False,
                                                              "position": position})

        def norms(i):
            return {"input": PartSpec("rmsnorm", f"l{i}.n1.", norm), "post_mixer": PartSpec("rmsnorm", f"l{i}.n2.", norm)}

        layers = (
            LayerSpec("prenorm", attention(0, PartSpec("test_interleaved_rope", "", {"head_dim": 16, "base": 500.0})),
                      PartSpec("test_top1_experts", "l0.moe.", {"hidden_size": c["hidden"], "experts": c["experts"], "expert_inter": c["expert_inter"]}), norms(0)),
            LayerSpec("prenorm", attention(1, PartSpec("rope", "", {"head_dim": 16, "base": 1e4, "max_positions": c["max_positions"]})),
                      PartSpec("swiglu", "l1.mlp.", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]}), norms(1)),
        )
        return ModelSpec("TestRoutedLM", c["hidden"], c["vocab"], c["max_positions"], PartSpec("token_embedding", "embed.", sizes), layers,
                         (Run(0), Run(1)), PartSpec("rmsnorm", "norm.", norm), PartSpec("linear_head", "head.", {**sizes, "tied": False}))

    register_feed_forward("test_top1_experts", TopOneExperts)
    register_position("test_interleaved_rope", InterleavedRotary)
    register_architecture(Architecture("TestRoutedLM", lambda document: dict(document), spec, lambda config: dict(config)))


def routed_plain(c, w, ids):
    w = {k: v.double() for k, v in w.items()}
    t = len(ids)
    positions = torch.arange(t)
    h = plain.embedding(w["embed.weight"], torch.tensor(ids))

    def interleaved(x):
        inv = 500.0 ** (-torch.arange(0, 16, 2, dtype=torch.float64) / 16)
        angle = positions.double()[:, None] * inv[None]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
        pairs = x.reshape(t, x.shape[1], 8, 2)
        return torch.stack([pairs[..., 0] * cos - pairs[..., 1] * sin, pairs[..., 1] * cos + pairs[..., 0] * sin], dim=-1).reshape(x.shape)

    for i in range(2):
        x = plain.rmsnorm(h, w[f"l{i}.n1.weight"], c["eps"])
        q = plain.linear(x, w[f"l{i}.attn.q_proj.weight"]).view(t, 4, 16)
        k = plain.linear(x, w[f"l{i}.attn.k_proj.weight"]).view(t, 2, 16)
        v = plain.linear(x, w[f"l{i}.attn.v_proj.weight"]).view(t, 2, 16)
        if i == 0:
            q, k = interleaved(q), interleaved(k)
        else:
            cos, sin = plain.rope_tables(positions, 16, 1e4)
            q, k = plain.rope(q, cos, sin), plain.rope(k, cos, sin)
        a = plain.attention(q, k, v, positions, positions, 0.25)
        h = h + plain.linear(a.reshape(t, -1), w[f"l{i}.attn.o_proj.weight"])
        x = plain.rmsnorm(h, w[f"l{i}.n2.weight"], c["eps"])
        if i == 0:
            probs = torch.softmax(x @ w["l0.moe.router.weight"].t(), dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros_like(x)
            for tok in range(t):
                e = int(choice[tok])
                out[tok] = (torch.nn.functional.gelu(x[tok] @ w["l0.moe.w1"][e].t()) @ w["l0.moe.w2"][e].t()) * weight[tok]
            h = h + out
        else:
            h = h + plain.swiglu_mlp(x, w["l1.mlp.gate_proj.weight"], w["l1.mlp.up_proj.weight"], w["l1.mlp.down_proj.weight"])
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], c["eps"]), w["head.weight"])


def test_a_routed_feed_forward_and_another_position_encoding(tmp_path):
    from hyperion_b200.api import Engine
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.weights import read_all, write_model_folder

    register_routed()
    folder = write_model_folder(tmp_path / "routed", "TestRoutedLM", ROUTED, seed=12, std=0.15)
    weights = read_all(folder)
    assert weights["l0.moe.w1"].shape == (4, 40, 64) and "l0.attn.q_proj.bias" not in weights
    g = torch.Generator().manual_seed(2)
    a, b = (torch.randint(0, ROUTED["vocab"], (n,), generator=g).tolist() for n in (60, 33))
    want_a, want_b = routed_plain(ROUTED, weights, a).numpy(), routed_plain(ROUTED, weights, b).numpy()
    engine = Engine.from_folder(folder, dtype="float32", page_size=8, max_tokens=128, max_requests=2)
    got = [engine.step([StepEntry("a", a[:25], list(range(25)))]).cpu().numpy()]
    mixed = engine.step([StepEntry("a", a[25:26], [0]), StepEntry("b", b, list(range(33)))]).cpu().numpy()
    got.append(mixed[:1])
    got.append(engine.step([StepEntry("a", a[26:], list(range(34)))]).cpu().numpy())
    assert np.abs(np.concatenate(got) - want_a).max() <= 1e-4 * np.abs(want_a).max()
    assert np.abs(mixed[1:] - want_b).max() <= 1e-4 * np.abs(want_b).max()


# ------------------------------------------------------------------------------------------------
# A toy mixer whose paged payload is one latent vector per token (not keys and values of heads): it states the shape,
# the cache manager sizes pages from it, the step hands it its pages and block table.  Nothing in the package knows it.
LATENT = {"architectures": ["TestLatentLM"], "hidden": 136, "vocab": 89, "inter": 152, "latent": 24, "eps": 1e-6, "max_positions": 256}


def register_latent():
    from hyperion_b200.models import Architecture, register_architecture
    from hyperion_b200.parts import MIXERS, LayerSpec, Mixer, ModelSpec, PagedTokens, PartSpec, Run, WeightSpec, register_mixer

    if "test_latent_attention" in MIXERS:  # the test runs once per element type
        return

    class LatentAttention(Mixer):
        """c_t = x_t W_c is kept per token; y_t = (sum_j softmax_j(q_t . c_j) c_j) W_o over j <= t with q_t = x_t W_q."""

        def __init__(self, spec, build):
            super().__init__(spec, build)
            self.hidden, self.latent = spec.params["hidden_size"], spec.params["latent"]

        def weights(self):
            return {"c.weight": WeightSpec((self.latent, self.hidden)), "q.weight": WeightSpec((self.latent, self.hidden)),
                    "o.weight": WeightSpec((self.hidden, self.latent))}

        def load(self, tensors):
            self.w_c, self.w_q, self.w_o = (tensors[n].float() for n in ("c.weight", "q.weight", "o.weight"))

        def cache_request(self):
            return PagedTokens(inner=(self.latent,), dtype=torch.float32)

        def forward(self, x, step, cache, own_cache):
            # everything that changes from step to step is read on the device: positions, rows, block tables
            pages, page_size, latent = cache.storage.shape
            xf = x.float()
            c, q = xf @ self.w_c.t(), xf @ self.w_q.t()
            rows, positions = step.token_row.long(), step.positions.long()
            page = cache.block_table[rows, positions // page_size].long()
            cache.storage[page, positions % page_size] = c
            table = cache.block_table[rows].long()  # [tokens, width]
            keys = cache.storage[table.clamp(min=0)].reshape(len(rows), -1, latent)  # every slot the row's table names
            slot_position = torch.arange(keys.shape[1], device=x.device)[None, :]
            scores = torch.einsum("tl,tsl->ts", q, keys).masked_fill(slot_position > positions[:, None], float("-inf"))
            mixed = torch.einsum("ts,tsl->tl", torch.softmax(scores, dim=-1), torch.nan_to_num(keys))
            return (mixed @ self.w_o.t()).to(self.dtype)

    def spec(c):
        sizes = {"vocab_size": c["vocab"], "hidden_size": c["hidden"]}
        norm = {"hidden_size": c["hidden"], "eps": c["eps"]}
        layers = tuple(LayerSpec("prenorm", PartSpec("test_latent_attention", f"l{i}.mix.", {"hidden_size": c["hidden"], "latent": c["latent"]}),
                                 PartSpec("swiglu", f"l{i}.mlp.", {"hidden_size": c["hidden"], "intermediate_size": c["inter"]}),
                                 {"input": PartSpec("rmsnorm", f"l{i}.n1.", norm), "post_mixer": PartSpec("rmsnorm", f"l{i}.n2.", norm)})
                       for i in range(2))
        return ModelSpec("TestLatentLM", c["hidden"], c["vocab"], c["max_positions"], PartSpec("token_embedding", "embed.", sizes), layers,
                         (Run(0), Run(1)), PartSpec("rmsnorm", "norm.", norm), PartSpec("linear_head", "head.", {**sizes, "tied": True}))

    register_mixer("test_latent_attention", LatentAttention)
    register_architecture(Architecture("TestLatentLM", lambda document: dict(document), spec, lambda config: dict(config)))


def latent_plain(c, w, ids, stored=lambda x: x):
    """Whole sequence in float64.  ``stored``: applied where the engine stores an activation in its element type (the
    norms' outputs, the mixer's and the feed-forward's results and what lies between their products): the identity for the
    exact model, a rounding to bfloat16 to measure what that storage costs this model."""
    w = {k: v.double() for k, v in w.items()}
    t = len(ids)
    h = plain.embedding(w["embed.weight"], torch.tensor(ids))
    causal = torch.arange(t)[None, :] <= torch.arange(t)[:, None]
    for i in range(2):
        x = stored(plain.rmsnorm(h, w[f"l{i}.n1.weight"], c["eps"]))
        latent, q = x @ w[f"l{i}.mix.c.weight"].t(), x @ w[f"l{i}.mix.q.weight"].t()
        probs = torch.softmax((q @ latent.t()).masked_fill(~causal, float("-inf")), dim=-1)
        h = h + stored((probs @ latent) @ w[f"l{i}.mix.o.weight"].t())
        x = stored(plain.rmsnorm(h, w[f"l{i}.n2.weight"], c["eps"]))
        gate, up = stored(x @ w[f"l{i}.mlp.gate_proj.weight"].t()), stored(x @ w[f"l{i}.mlp.up_proj.weight"].t())
        h = h + stored(stored(gate / (1.0 + torch.exp(-gate)) * up) @ w[f"l{i}.mlp.down_proj.weight"].t())
    return plain.linear(stored(plain.rmsnorm(h, w["norm.weight"], c["eps"])), w["embed.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_mixer_that_keeps_one_latent_per_token_in_pages(tmp_path, dtype):
    from hyperion_b200.api import Engine
    from hyperion_b200.engine.batch import StepEntry
    from hyperion_b200.sampling import SamplingParams
    from hyperion_b200.weights import read_all, write_model_folder

    register_latent()
    folder = write_model_folder(tmp_path / "latent", "TestLatentLM", LATENT, seed=21, std=0.07)
    weights = read_all(folder)
    engine = Engine.from_folder(folder, dtype=dtype, page_size=8, max_tokens=96, max_requests=3)
    cache = engine.cache
    assert len(cache.paged) == 1 and cache.paged[0].users == [0, 1] and cache.paged[0].storage.shape == (2, 12, 8, LATENT["latent"])
    assert cache.paged[0].storage.dtype == torch.float32 and cache.bytes_per_token() == 2 * LATENT["latent"] * 4
    g = torch.Generator().manual_seed(3)
    requests = {name: torch.randint(0, LATENT["vocab"], (n,), generator=g).tolist() for name, n in (("a", 50), ("b", 21), ("c", 40))}
    want = {name: latent_plain(LATENT, weights, ids).numpy() for name, ids in requests.items()}
    if dtype == "float32":
        tolerance = 1e-4
    else:
        # This mixer's keys are its values, which makes it touchy: what rounding its activations to bfloat16 costs is measured
        # on the plain model, and the engine may be off by that drift times a margin (the rule of the reference's oracle,
        # helios/crates/helios-hal/src/oracle.rs:186-217: the reference run's own bfloat16 deviation times 1.5).
        as_bfloat16 = lambda x: x.to(torch.bfloat16).double()
        drift = max(float(np.abs(latent_plain(LATENT, weights, ids, as_bfloat16).numpy() - want[name]).max() / np.abs(want[name]).max())
                    for name, ids in requests.items())
        tolerance = 1.5 * drift
        assert 0.005 < tolerance < 0.1, tolerance
    fed = {name: 0 for name in requests}
    order, sizes, k = ["a", "b"], [7, 2, 13, 1, 1, 20, 3], 0
    while order:
        entries = []
        for name in list(order):
            n = min(sizes[k % len(sizes)], len(requests[name]) - fed[name])
            k += 1
            entries.append(StepEntry(name, requests[name][fed[name]:fed[name] + n], list(range(n))))
        logits = engine.step(entries).float().cpu().numpy()
        row = 0
        for entry in entries:
            n = len(entry.tokens)
            ref = want[entry.request][fed[entry.request]:fed[entry.request] + n]
            error = np.abs(logits[row:row + n] - ref).max() / np.abs(want[entry.request]).max()
            assert error <= tolerance, (entry.request, fed[entry.request], float(error))
            row += n
            fed[entry.request] += n
            if fed[entry.request] == len(requests[entry.request]):
                engine.finish(entry.request)
                order.remove(entry.request)
                if entry.request == "b":
                    order.append("c")  # on the pages b gave back: 50 + 21 + 40 tokens do not fit 96 at once
        cache.check()
    assert cache.free_pages(0) == cache.num_pages
    # through the scheduler too: admission reserves pages of this group by its own need
    tokens = engine.generate([requests["b"]], SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True), lookahead=False)
    ref = latent_plain(LATENT, weights, requests["b"] + tokens[0]).numpy()
    for i, token in enumerate(tokens[0]):
        row = ref[len(requests["b"]) + i - 1]
        assert row.max() - row[token] <= 2 * tolerance * np.abs(row).max()
