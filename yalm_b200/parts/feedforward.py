"""SwiGLU feed-forward: x += W2 (silu(W1 h) * (W3 h)), silu(z) = z/(1+exp(-z))
(infer.cpp:356-385, infer.cu:610-634, 936-960).  Gate and up matrices are
kept as one matrix so that one product and its epilogue serve both: when the
width allows it, 16 gate rows are followed by the 16 up rows of the same features
(a tile of the product then holds both halves of each feature); otherwise the up
matrix simply follows the gate matrix.
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
        self.paired = False
        self.w_down = None

    def tensor_needs(self):
        return {"gate": TensorNeed((self.F, self.D)), "up": TensorNeed((self.F, self.D)),
                "down": TensorNeed((self.D, self.F))}

    def bind(self, tensors) -> None:
        parts = [tensors["gate"], tensors["up"]]
        if any(p.dtype == torch.float32 for p in parts):
            parts = [p.to(torch.float32) for p in parts]
        self.paired = self.F % 16 == 0
        if self.paired:
            g, u = (p.reshape(self.F // 16, 16, self.D) for p in parts)
            self.w_gate_up = self.rt.matrix(torch.stack([g, u], 1).reshape(2 * self.F, self.D))
        else:
            self.w_gate_up = self.rt.matrix(torch.cat(parts, 0))
        self.w_down = self.rt.matrix(tensors["down"])

    def flops(self, q_lens, past) -> float:
        return 2.0 * sum(q_lens) * 3 * self.F * self.D

    def forward(self, h, batch, stream) -> None:
        act = self.rt.buffer("ffn_act", (h.shape[0], self.F), self.rt.dtype)
        matmul_silu_mul(self.rt, h, self.w_gate_up, act, self.paired)
        stream.add_linear(act, self.w_down)
