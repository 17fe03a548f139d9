"""RMSNorm: o = x * w / sqrt(mean(x^2) + eps), all in 32 bits; the weight
multiplies (no 1 + w), as the reference computes it (infer.cpp:136-146,
infer.cu:525-539)."""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights import TensorNeed
from .base import ResidualStream, register_norm


@register_norm("rmsnorm")
class RMSNorm:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return {"weight": TensorNeed((self.size,), init="ones")}

    def bind(self, tensors) -> None:
        self.weight = self.rt.vector(tensors["weight"])

    def __call__(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None,
                 n_rows: Optional[int] = None, name: str = "normed") -> torch.Tensor:
        n = stream.x.shape[0] if rows is None else int(n_rows)
        out = self.rt.buffer(name, (n, self.size), self.rt.dtype)
        ops.rmsnorm(stream.x, self.weight, out, self.eps, partials=stream.pending,
                    n_partials=stream.n_pending, rows=rows)
        if rows is None:
            stream.pending, stream.n_pending = None, 0     # folded into x by the kernel
        return out
