"""A plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, no batching,
one function per part, torch on the CPU in float64 (or any dtype asked for).

It shares no code with the package.  The reference's own model code is Rust and CUDA and cannot be
compiled or run here, so this file rests on the reference's formulas, cited per function; the
reference's committed float32 oracle of a tiny checkpoint anchors it (tests/golden/).  The
reference stores bfloat16 and rounds after every operation; this implementation does not round, it
is the exact arithmetic both the 32-bit and the bfloat16 engine paths are compared with.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64,
          "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: Path) -> dict[str, torch.Tensor]:
    """One safetensors file: 8-byte length, JSON header, payload at 8 + length + offset
    (helios/crates/helios-hal/src/weights_plan.rs:38-46)."""
    blob = Path(path).read_bytes()
    (length,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + length])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        begin, end = meta["data_offsets"]
        raw = bytearray(blob[8 + length + begin : 8 + length + end])
        out[name] = torch.frombuffer(raw, dtype=DTYPES[meta["dtype"]]).reshape(meta["shape"]).clone()
    return out


def read_model_folder(folder: Path) -> tuple[dict, dict[str, torch.Tensor]]:
    """config.json and all tensors of a folder (single file or sharded index)."""
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    tensors: dict[str, torch.Tensor] = {}
    if (folder / "model.safetensors").is_file():
        tensors = read_safetensors(folder / "model.safetensors")
    else:
        index = json.loads((folder / "model.safetensors.index.json").read_text())
        for shard in sorted(set(index["weight_map"].values())):
            tensors.update(read_safetensors(folder / shard))
    return config, tensors


def dims(config: dict) -> dict:
    """Sizes from config.json with the reference's defaults
    (ignition/src/hyperion_ignition/compiler/model_config.py:124-135, :83-93)."""
    heads = config["num_attention_heads"]
    theta = config["rope_theta"] if "rope_theta" in config else config["rope_parameters"]["rope_theta"]
    return {
        "layers": config["num_hidden_layers"], "hidden": config["hidden_size"], "inter": config["intermediate_size"],
        "heads": heads, "kv_heads": config.get("num_key_value_heads", heads),
        "head_dim": config.get("head_dim", config["hidden_size"] // heads), "vocab": config["vocab_size"],
        "theta": float(theta), "eps": float(config["rms_norm_eps"]), "tied": bool(config["tie_word_embeddings"]),
    }


def embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """h[t] = table[ids[t]] (helios/crates/helios-hal/kernels/elementwise.cu:13-19)."""
    return table[ids.long()]


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + eps) * weight; the weight multiplies after the normalisation, no 1 + w
    (helios/crates/helios-hal/src/reference.rs:160-174; kernels/rmsnorm.cu:22-58)."""
    inv = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * inv * weight


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """y = x W^T (+ b), W stored [out, in] (helios/crates/helios-hal/src/reference.rs:24-41; bias added
    to the float accumulator, kernels/elementwise.cu:131-142)."""
    y = x @ weight.t()
    return y + bias if bias is not None else y


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype=torch.float64) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin of position * theta^(-2i/d), i < d/2, computed in float64
    (helios/crates/helios-hal/src/reference.rs:71-87)."""
    i = torch.arange(head_dim // 2, dtype=torch.float64, device=positions.device)
    inv_freq = theta ** (-2.0 * i / head_dim)
    angle = positions.to(torch.float64)[:, None] * inv_freq[None, :]
    return angle.cos().to(dtype), angle.sin().to(dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """rotate_half convention on x [tokens, heads, d]: first half x1 c - x2 s, second half x2 c + x1 s
    (helios/crates/helios-hal/src/reference.rs:91-109; kernels/elementwise.cu:42-56)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_positions: torch.Tensor, k_positions: torch.Tensor,
              scale: float, window: int | None = None) -> torch.Tensor:
    """Causal grouped-query attention: query head h uses kv head h // (heads / kv_heads); key j is
    visible to a query at position p when j <= p (and j > p - window when a window is set); softmax of
    (q.k) * scale; weighted sum of the values (helios/crates/helios-hal/src/reference.rs:118-156).
    q [T, heads, d]; k, v [S, kv_heads, d]; returns [T, heads, d]."""
    heads, kv_heads = q.shape[1], k.shape[1]
    group = heads // kv_heads
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("thd,shd->hts", q, kk) * scale
    visible = k_positions[None, :] <= q_positions[:, None]
    if window:
        visible &= k_positions[None, :] > q_positions[:, None] - window
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hts,shd->thd", probs, vv)


def swiglu_mlp(x: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), silu(g) = g / (1 + exp(-g)), no biases
    (helios/crates/helios-hal/src/reference.rs:56-66; backends/hopper_sm90/session.rs:779-793)."""
    g = linear(x, gate_w)
    return linear(g / (1.0 + torch.exp(-g)) * linear(x, up_w), down_w)


def attention_block(x: torch.Tensor, w: dict[str, torch.Tensor], prefix: str, d: dict, positions: torch.Tensor,
                    window: int | None = None) -> torch.Tensor:
    """q/k/v projections with bias, RoPE on q and k, attention, output projection without bias
    (helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:716-772)."""
    t = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"]).view(t, d["heads"], d["head_dim"])
    k = linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"]).view(t, d["kv_heads"], d["head_dim"])
    v = linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"]).view(t, d["kv_heads"], d["head_dim"])
    cos, sin = rope_tables(positions, d["head_dim"], d["theta"], x.dtype)
    q, k = rope(q, cos, sin), rope(k, cos, sin)
    a = attention(q, k, v, positions, positions, 1.0 / math.sqrt(d["head_dim"]), window)
    return linear(a.reshape(t, -1), w[prefix + "o_proj.weight"])


def decoder_layer(h: torch.Tensor, w: dict[str, torch.Tensor], layer: int, d: dict, positions: torch.Tensor) -> torch.Tensor:
    """Pre-norm block: h += attn(norm(h)); h += mlp(norm(h))
    (helios/crates/helios-hal/src/backends/hopper_sm90/session.rs:710-799)."""
    p = f"model.layers.{layer}."
    h = h + attention_block(rmsnorm(h, w[p + "input_layernorm.weight"], d["eps"]), w, p + "self_attn.", d, positions)
    x = rmsnorm(h, w[p + "post_attention_layernorm.weight"], d["eps"])
    return h + swiglu_mlp(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def forward(config: dict, weights: dict[str, torch.Tensor], ids, dtype=torch.float64, device="cpu") -> torch.Tensor:
    """Logits [tokens, vocab] of one whole sequence starting at position 0: embedding, the layers,
    final norm, LM head (lm_head.weight, or the embedding table when tied:
    helios/crates/helios-hal/src/backends/hopper_sm90/forward.rs:45-51; session.rs:807-810).
    ``device``: where torch does this arithmetic (the CPU, or a GPU for models of real widths: the
    same functions in the same 64-bit type)."""
    d = dims(config)
    w = {name: tensor.to(device=device, dtype=dtype) for name, tensor in weights.items() if tensor.is_floating_point()}
    ids = torch.as_tensor(ids, dtype=torch.long, device=device)
    positions = torch.arange(ids.numel(), device=device)
    h = embedding(w["model.embed_tokens.weight"], ids)
    for layer in range(d["layers"]):
        h = decoder_layer(h, w, layer, d, positions)
    x = rmsnorm(h, w["model.norm.weight"], d["eps"])
    head = w["model.embed_tokens.weight"] if d["tied"] else w["lm_head.weight"]
    return linear(x, head)


def greedy(config: dict, weights: dict[str, torch.Tensor], prompt: list[int], steps: int, dtype=torch.float64) -> list[int]:
    """Argmax continuation, lowest index on ties (helios/crates/helios-hal/src/sampling.rs:50-58)."""
    ids = list(prompt)
    for _ in range(steps):
        logits = forward(config, weights, ids, dtype)[-1]
        ids.append(int(torch.argmax(logits)))
    return ids[len(prompt):]
