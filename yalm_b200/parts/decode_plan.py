"""The decode attention's choice between its two block shapes, by an estimate
of how long the grid takes.

The tensor-core decode kernel exists with four warps per block and with two.
Every warp streams keys and values through a ring of its own, so a two-warp
block pulls half of what a four-warp block does, needs half the shared memory,
and two of them fit where one four-warp block does.  Which is faster depends on
how the blocks fall on the SMs:

* few long blocks (20 sequences of 2,048 keys, 8 kv heads: 160 blocks): four
  warps run 148 blocks and then 12 while 136 SMs idle; two warps run all 160 at
  once (4.21 against 3.93 ms per step at 7B sizes);
* ragged lengths, longest first, one to three waves: the short blocks fill the
  SMs that long four-warp blocks leave, and a two-warp block of the longest
  sequence is what everything waits for (32 sequences of 64 to 2,048 keys:
  3.60 against 3.90 ms);
* many waves: blocks' starts and ends overlap other blocks' copies only when
  two blocks share an SM (64 sequences: 4.99 against 4.83 ms).

The estimate is a small event simulation: blocks take free slots in launch
order; a block spends ``START`` microseconds before its first bytes and ``END``
after its last; in between all streaming blocks share the memory's rate
equally, each capped at ``WARP_RATE`` per warp.  The constants were fitted to
92 measured pairs of step times (7B and Llama-3.2-1B sizes; 19 to 128
sequences; contexts equal, ragged, short and long).  The estimate overstates
the difference by about half, so the two-warp shape is taken only where it
wins by 5 %; with that (and lengths rounded as ``rounded`` does) the choice is
the faster shape in 71 of the 76 pairs that differ by more than a microsecond
per layer, and each of the five misses forgoes 1 to 3 us.
"""
from __future__ import annotations

import functools
import heapq
from typing import Sequence, Tuple

START_US = 1.0            # slot, position, page, first copies on their way
END_US = 3.0              # the warps' merge through shared memory, the output, the block's exit
WARP_RATE = 16384.0       # bytes per microsecond one warp's ring sustains (two units in flight)
MEMORY_RATE = 6.2e6       # bytes per microsecond all blocks together
SHARED_PER_SM = 227 * 1024
MOST_BLOCKS = 4096        # beyond this the grid has many waves anyway: no simulation
MARGIN = 0.95


def ring_bytes(warps: int, head_dim_padded: int) -> int:
    """Shared memory of a block: 16 query rows and, per warp, three stages of 32 keys and 32 values."""
    return (16 + warps * 3 * 2 * 32) * head_dim_padded * 2


def grid_time(block_bytes: Sequence[float], slots: int, block_rate: float,
              memory_rate: float = MEMORY_RATE) -> float:
    """Microseconds until the last block has ended."""
    timers = []                       # (time, 0: starts to stream / 1: has ended, bytes)
    finish = []                       # bytes every streaming block has been served when this one is through
    served = 0.0                      # bytes served to each streaming block so far
    t = 0.0
    nxt, free, done, n = 0, slots, 0, len(block_bytes)
    while done < n:
        while free > 0 and nxt < n:
            heapq.heappush(timers, (t + START_US, 0, block_bytes[nxt]))
            nxt += 1
            free -= 1
        rate = min(block_rate, memory_rate / len(finish)) if finish else 0.0
        to_finish = (finish[0] - served) / rate if finish else float("inf")
        to_timer = timers[0][0] - t if timers else float("inf")
        if to_timer <= to_finish:
            served += rate * to_timer
            t += to_timer
            _, kind, nbytes = heapq.heappop(timers)
            if kind == 0:
                heapq.heappush(finish, served + nbytes)
            else:
                done += 1
                free += 1
        else:
            served = heapq.heappop(finish)
            t += to_finish
            heapq.heappush(timers, (t + END_US, 1, 0.0))
    return t


def rounded(chunks: Sequence[int]) -> Tuple[int, ...]:
    """Chunk counts, the longer ones rounded up (to 2 from 16 chunks on, to 4 from 32): long
    sequences that grow token by token then ask for a new estimate only now and then."""
    return tuple(c if c <= 16 else -(-c // 2) * 2 if c <= 32 else -(-c // 4) * 4 for c in chunks)


@functools.lru_cache(maxsize=256)
def decode_warps(chunks: Tuple[int, ...], groups: int, head_dim: int, sm_count: int,
                 element_size: int = 2) -> int:
    """4 or 2: warps per block for a grid of whole-sequence blocks.  ``chunks``: 64-key chunks
    of each sequence, in launch order; ``groups`` blocks per sequence.  (Every attention layer
    of a model asks the same question in a step: the answers are kept.)"""
    head_dim_padded = 64 if head_dim <= 64 else 128
    n_blocks = groups * len(chunks)
    slots4 = sm_count * max(1, SHARED_PER_SM // ring_bytes(4, head_dim_padded))
    slots2 = sm_count * max(1, SHARED_PER_SM // ring_bytes(2, head_dim_padded))
    if n_blocks <= slots4:
        return 4
    if n_blocks > MOST_BLOCKS:
        return 2
    chunk_bytes = 64.0 * 2 * head_dim * element_size
    blocks = [c * chunk_bytes for c in chunks for _ in range(groups)]
    t4 = grid_time(blocks, slots4, 4 * WARP_RATE)
    t2 = grid_time(blocks, slots2, 2 * WARP_RATE)
    return 2 if t2 < MARGIN * t4 else 4
