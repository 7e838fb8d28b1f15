"""Token embedding and output head.

h[t] = table[ids[t]] (helios/crates/helios-hal/kernels/elementwise.cu:13-19); logits = x head^T kept in
float, where head is ``lm_head.weight`` or, with tied embeddings, the embedding table
(helios/crates/helios-hal/src/backends/hopper_sm90/forward.rs:45-51, session.rs:844-848).
Parameters: ``vocab_size``, ``hidden_size``; the head also ``tied`` (then it owns no tensor and is
handed the embedding's table).
"""
from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from .base import BuildContext, Embedding, Head, WeightSpec, register_embedding, register_head
from .spec import PartSpec


class TokenEmbedding(Embedding):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])

    def weights(self):
        return {"weight": WeightSpec((self.vocab, self.hidden))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors["weight"].contiguous()

    def kernel_modules(self):
        return [("elementwise", {})]

    def forward(self, token_ids):
        return ops.embedding(self.table, token_ids)

    def shared_table(self):
        return self.table


class LinearHead(Head):
    def __init__(self, spec: PartSpec, build: BuildContext):
        super().__init__(spec, build)
        self.vocab = int(spec.params["vocab_size"])
        self.hidden = int(spec.params["hidden_size"])
        self.tied = bool(spec.params.get("tied", False))
        self.weight = None

    def weights(self):
        return {} if self.tied else {"weight": WeightSpec((self.vocab, self.hidden))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def wants_shared_table(self) -> bool:
        return self.tied

    def use_shared_table(self, table: torch.Tensor) -> None:
        if tuple(table.shape) != (self.vocab, self.hidden):
            raise ValueError(f"the tied head wants a table of {(self.vocab, self.hidden)}, the embedding shares {tuple(table.shape)}")
        self.weight = table

    def kernel_modules(self):
        return [("sgemm_f32", {}) if self.dtype == torch.float32 else ("gemm_tcgen05", {})]

    def forward(self, x):
        return ops.linear(x, self.weight, None, torch.float32)


register_embedding("token_embedding", TokenEmbedding)
register_head("linear_head", LinearHead)
