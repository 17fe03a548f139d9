"""Sampling.  The device kernel lives in csrc/sampling.cu (greedy: first maximal index;
temperature: inverse CDF of exp((l - max)/T) with a counter-based uniform number keyed by
(seed, request, position); the reference: sampler.cpp:27-64).  This module is what the engine
calls: the launch, the two words a captured decode step reads seed and temperature from, and
the generator's host-side twin, with which a caller can reproduce the number the device
draws for a token.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..csrc import ops


def sample(logits: torch.Tensor, temperature: float, seed: int, row_key: torch.Tensor,
           seq_slot: torch.Tensor, slot_pos: torch.Tensor, out_tokens: torch.Tensor,
           params: Optional[torch.Tensor] = None) -> None:
    """One token per row of ``logits`` [rows, vocab] into ``out_tokens``: the first maximal
    index at temperature 0, else a draw keyed by (seed, row_key[r], the position after
    slot_pos[seq_slot[r]]).  With ``params`` (``device_params`` on the device) the kernel
    reads seed and temperature from there instead of from the arguments."""
    ops.sample(logits, temperature, seed, row_key, seq_slot, slot_pos, out_tokens, params)


def device_params(temperature: float, seed: int) -> Tuple[int, int]:
    """The two 64-bit words (seed, temperature bits) that ``sample`` reads from ``params``."""
    return ops.sampling_params(temperature, seed)


def uniform01(seed: int, key: int, position: int) -> float:
    """The number in [0, 1) that the device draws for (seed, request key,
    position of the new token)."""
    return ops.uniform01(seed, key, position)
