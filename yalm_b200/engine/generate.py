"""The generation loop: batches of unequal prompts, stop tokens, sequences that
end earlier than their batch, and as many batches one after another as there
are requests.

The reference's loop serves one sequence: prefill, then sample -> append ->
stop check -> forward (main.cpp:104-129); the stop token is part of the output
and is not forwarded.  Here the same decisions are taken per sequence of a
batch.  The loop talks to the device through a small backend interface, so its
decisions can be tested without one:

    backend.max_batch                       -> most sequences in one batch
    backend.context                         -> most positions of one sequence
    backend.begin(prompts, keys)            -> (handle, first sampled token per prompt)
    backend.decode(handle, active, tokens)  -> next sampled token per active sequence
    backend.end(handle)                     -> gives the batch's slots back
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence


@dataclass
class Completion:
    prompt_len: int
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "stop" | "length" | "context"


def plan_batches(n_requests: int, max_batch: int) -> List[List[int]]:
    """Request indices per batch, in order, at most ``max_batch`` each."""
    if max_batch <= 0:
        raise ValueError("max_batch must be positive")
    return [list(range(i, min(i + max_batch, n_requests))) for i in range(0, n_requests, max_batch)]


def run_generation(backend, prompts: Sequence[Sequence[int]], max_new_tokens: int,
                   stop_ids: Sequence[int] = (), on_token=None) -> List[Completion]:
    """Greedy or sampled continuation of every prompt (the backend samples).
    ``max_new_tokens < 0`` means: until a stop token or the context's end."""
    stop = set(int(t) for t in stop_ids)
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) > backend.context:
            raise ValueError(f"prompt {i} has {len(p)} tokens; the context is {backend.context}")
    results = [Completion(prompt_len=len(p)) for p in prompts]
    if max_new_tokens == 0:
        for r in results:
            r.finish_reason = "length"
        return results
    for batch_ids in plan_batches(len(prompts), backend.max_batch):
        handle, first = backend.begin([list(prompts[i]) for i in batch_ids], list(batch_ids))
        try:
            active = list(range(len(batch_ids)))      # indices into this batch
            new_tokens = list(first)
            while active:
                still, carry = [], []
                for j, tok in zip(active, new_tokens):
                    r = results[batch_ids[j]]
                    r.tokens.append(int(tok))
                    if on_token is not None:
                        on_token(batch_ids[j], int(tok))
                    if int(tok) in stop:
                        r.finish_reason = "stop"
                    elif 0 <= max_new_tokens <= len(r.tokens):
                        r.finish_reason = "length"
                    elif r.prompt_len + len(r.tokens) > backend.context:
                        # forwarding the new token would need a position the context does not have
                        r.finish_reason = "context"
                    else:
                        still.append(j)
                        carry.append(int(tok))
                active = still
                if active:
                    new_tokens = backend.decode(handle, active, carry)
        finally:
            backend.end(handle)
    return results
