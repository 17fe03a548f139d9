"""Sampling.  The device kernels live in csrc/sampling.cu (greedy: first
maximal index; temperature: inverse CDF of exp((l - max)/T), sampler.cpp:27-64);
this module is their host-side face: the counter-based uniform generator and a
host implementation of the same rule for callers that hold logits on the CPU.
"""
from __future__ import annotations

import torch


def uniform01(seed: int, key: int, position: int) -> float:
    """The number in [0, 1) that the device draws for (seed, request key,
    position of the new token)."""
    from ..csrc import ops
    return ops.uniform01(seed, key, position)


def sample_host(logits: torch.Tensor, temperature: float, u: float) -> int:
    """The kernels' rule on a CPU row of logits."""
    if temperature == 0.0:
        return int(torch.argmax(logits).item()) if logits.numel() else 0
    l = logits.double()
    e = torch.exp((l - l.max()) / temperature)
    c = torch.cumsum(e, 0)
    idx = int(torch.searchsorted(c, torch.tensor(u * float(c[-1]), dtype=torch.float64)).item())
    return min(idx, logits.numel() - 1)
