"""Token embedding (x = float(E[token]), infer.cpp:454-475) and the output
head (logits = Wcls x, the embedding matrix when tied, model.cpp:389-398)."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..weights import TensorNeed
from .base import register_embedding, register_head
from .linear import matmul_store


@register_embedding("embedding")
class Embedding:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.size = int(params["size"])
        self.table = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.vocab, self.size))}

    def bind(self, tensors) -> None:
        self.table = self.rt.matrix(tensors["weight"], share=True)

    def forward(self, batch) -> torch.Tensor:
        x = self.rt.buffer("residual", (batch.n_tokens, self.size), torch.float32)
        ops.embed(batch.tokens, self.table, x, self.rt.status)
        return x


@register_head("linear_head")
class LinearHead:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.vocab = int(params["vocab_size"])
        self.size = int(params["size"])
        self.weight = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.vocab, self.size))}

    def bind(self, tensors) -> None:
        self.weight = self.rt.matrix(tensors["weight"], share=True)

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * self.vocab * self.size

    def forward(self, h: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        matmul_store(self.rt, h, self.weight, out)
        return out
