"""The batch of one step: the tokens of several sequences laid end to end
(ragged, no padding) with the index arrays the kernels need.

Device arrays (int32): ``tokens[N]``, ``token_seq[N]`` (which sequence a token
belongs to), ``q_start[B+1]`` (where each sequence's tokens begin) and
``seq_slot[B]`` (its cache slot).  A token's position is the slot's position
on the device plus its offset in the sequence, so nothing here changes between
decode steps of the same sequences except ``tokens``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    q_lens: List[int]
    slots: List[int]
    past: List[int]                       # each sequence's length before the step (host view)
    tokens: torch.Tensor
    token_seq: torch.Tensor
    q_start: torch.Tensor
    seq_slot: torch.Tensor
    want_rows: Optional[torch.Tensor] = None   # int32 flat token indices whose logits are wanted
    n_want: int = 0
    ctx_bound: int = 0                    # no sequence exceeds this many positions after the step
    notes: dict = field(default_factory=dict)  # what parts make once per step and share between layers

    @property
    def is_decode(self) -> bool:
        return all(q == 1 for q in self.q_lens)

    @property
    def max_context(self) -> int:
        return max(p + q for p, q in zip(self.past, self.q_lens))


def build_batch(token_lists: Sequence[Sequence[int]], slots: Sequence[int], past: Sequence[int],
                want: Sequence[Sequence[int]], device) -> StepBatch:
    """``want[b]`` lists offsets into sequence b's tokens whose logits are
    wanted.  All index arrays go to the device in one copy from pinned memory."""
    B = len(token_lists)
    q_lens = [len(t) for t in token_lists]
    N = sum(q_lens)
    q_start = [0]
    for q in q_lens:
        q_start.append(q_start[-1] + q)
    pieces, rows = [], []
    for b, toks in enumerate(token_lists):
        pieces.append(np.asarray(toks, dtype=np.int32))
        w = np.asarray(want[b], dtype=np.int64)
        if w.size:
            if int(w.min()) < 0 or int(w.max()) >= len(toks):
                bad = next(x for x in want[b] if not 0 <= x < len(toks))
                raise IndexError(f"sequence {b}: wanted place {bad} is outside its {len(toks)} tokens")
            rows.append((w + q_start[b]).astype(np.int32))
    rows = np.concatenate(rows) if rows else np.zeros(0, dtype=np.int32)
    tseq = np.repeat(np.arange(B, dtype=np.int32), q_lens)
    host = torch.from_numpy(np.concatenate(
        pieces + [tseq, np.asarray(q_start, dtype=np.int32), np.asarray(list(slots), dtype=np.int32), rows]))
    if torch.device(device).type == "cuda":
        host = host.pin_memory()
    dev = host.to(device, non_blocking=True)
    o = 0
    tokens = dev[o:o + N]; o += N
    token_seq = dev[o:o + N]; o += N
    qs = dev[o:o + B + 1]; o += B + 1
    seq_slot = dev[o:o + B]; o += B
    want_rows = dev[o:o + len(rows)]
    return StepBatch(n_tokens=N, n_seqs=B, q_lens=q_lens, slots=list(slots), past=list(past),
                     tokens=tokens, token_seq=token_seq, q_start=qs, seq_slot=seq_slot,
                     want_rows=want_rows, n_want=len(rows),
                     ctx_bound=max(p + q for p, q in zip(past, q_lens)))
