"""Position encodings.  A mixer owns one and calls
``rotate_and_store(qkv, n_partials, batch, view, q_out, kv_step, H, G, write_cache)``
after its q/k/v projection: the encoding rotates q and k, and the fused kernel
writes k and v into the cache on the way.

``rope``: pairs (i, i + head_dim/2) of each head are rotated by the angle
pos * inv_freq[i], computed in 32 bits inside the kernel.  The reference rotates
interleaved pairs of weights whose rows its packer permuted (infer.cpp:202-215,
convert.py:145-158); on unpermuted checkpoints that is this half-split pairing.
inv_freq[i] = theta^(-2i/head_dim), optionally rescaled by the llama3 rule
(long wavelengths divided by ``factor``, short ones kept, a linear blend
between), which the reference does not read.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..csrc import ops
from .base import register_position


def llama3_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    out = []
    for i in range(0, head_dim, 2):
        f = 1.0 / (float(theta) ** (i / head_dim))
        if scaling is not None:
            factor = float(scaling["factor"])
            low = float(scaling["low_freq_factor"])
            high = float(scaling["high_freq_factor"])
            orig = float(scaling["original_max_position_embeddings"])
            wavelen = 2.0 * math.pi / f
            if wavelen > orig / low:
                f = f / factor
            elif wavelen >= orig / high:
                s = (orig / wavelen - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64).to(torch.float32)


@register_position("rope")
class Rope:
    def __init__(self, params: dict, rt):
        self.rt = rt
        self.head_dim = int(params["head_dim"])
        if self.head_dim % 2:
            raise ValueError(f"rope needs an even head size, got {self.head_dim}")
        self.inv_freq = llama3_inv_freq(self.head_dim, float(params["theta"]),
                                        params.get("scaling")).to(rt.device)
        scaling = params.get("scaling")
        self._table_key = "rope_table_%d_%r_%r" % (
            self.head_dim, float(params["theta"]),
            None if scaling is None else tuple(sorted((k, str(v)) for k, v in scaling.items())))

    def step_table(self, batch, slot_pos) -> torch.Tensor:
        """(cos, sin) of every token's angle for every pair, float32 [tokens, head_dim/2, 2]:
        made once per step and shared by the layers whose encoding has the same constants,
        for a q/k/v product that rotates and stores in its own epilogue (an encoding
        without this method always gets ``rotate_and_store``)."""
        table = batch.notes.get(self._table_key)
        if table is None:
            table = self.rt.buffer(self._table_key, (batch.n_tokens, self.head_dim // 2, 2),
                                   torch.float32)
            ops.rope_table(self.inv_freq, batch, slot_pos, table)
            batch.notes[self._table_key] = table
        return table

    def rotate_and_store(self, qkv, n_partials, batch, view, q_out, kv_step, H, G,
                         write_cache=True) -> None:
        ops.rope_store(qkv, n_partials, self.inv_freq, batch, q_out, kv_step, view.k, view.v,
                       view.slot_pos, H, G, self.head_dim, view.capacity, write_cache,
                       pages=view.pages)
