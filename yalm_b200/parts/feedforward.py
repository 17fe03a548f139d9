"""SwiGLU feed-forward: x += W2 (silu(W1 h) * (W3 h)), silu(z) = z/(1+exp(-z))
(infer.cpp:356-385, infer.cu:610-634, 936-960).  Gate and up matrices are
stacked so that one product (and, with many tokens, one epilogue) serves both.
"""
from __future__ import annotations

import torch

from ..weights import TensorNeed
from .base import register_feed_forward
from .linear import matmul_silu_mul


@register_feed_forward("swiglu")
class SwiGLU:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.D = int(params["hidden_size"])
        self.F = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def tensor_needs(self):
        return {"gate": TensorNeed((self.F, self.D)), "up": TensorNeed((self.F, self.D)),
                "down": TensorNeed((self.D, self.F))}

    def bind(self, tensors) -> None:
        parts = [tensors["gate"], tensors["up"]]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.w_gate_up = self.rt.matrix(torch.cat(parts, 0))
        self.w_down = self.rt.matrix(tensors["down"])

    def forward(self, h, batch, stream) -> None:
        act = self.rt.buffer("ffn_act", (h.shape[0], self.F), self.rt.dtype)
        matmul_silu_mul(self.rt, h, self.w_gate_up, act)
        stream.add_linear(act, self.w_down)
