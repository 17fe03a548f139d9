"""Sampling.  The device kernel lives in csrc/sampling.cu (greedy: first
maximal index; temperature: inverse CDF of exp((l - max)/T), sampler.cpp:27-64);
this module is its host-side face: the counter-based uniform generator, so that a
caller can reproduce the number the device draws for a token.
"""
from __future__ import annotations


def uniform01(seed: int, key: int, position: int) -> float:
    """The number in [0, 1) that the device draws for (seed, request key,
    position of the new token)."""
    from ..csrc import ops
    return ops.uniform01(seed, key, position)
