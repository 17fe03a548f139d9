"""The step function: one batch of sequences, only the tokens it is given,
from the cache that earlier steps left, logits at the wanted places.

The reference's step is ``Model::forward(state, token, pos, mode)``: one token
of one sequence, logits or none (model.h:260, infer.cu:1103-1207).  Here a
step takes a ragged batch: all prompts of a batch at once, then one token per
sequence; a sequence's position lives in the cache's per-slot record on the
device and is advanced by the step itself.

Decode steps of a fixed set of sequences are captured once into a CUDA graph
(embedding to sampling) and replayed; the sampled token is written where the
next step's embedding reads it, so the device can decode on its own while the
host only reads tokens back.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache import Cache, CacheFull
from .. import sampling
from ..csrc import ops
from ..parts import Model
from .batch import StepBatch, build_batch


class StepError(RuntimeError):
    pass


class CacheMemoryError(StepError):
    """The cache that was asked for does not fit the device's free memory."""


class Engine:
    def __init__(self, model: Model, n_slots: int, context: int, max_tokens: Optional[int] = None):
        """``n_slots`` sequences may be live at once, each up to ``context`` positions.
        ``max_tokens``: the most tokens they hold together (each count rounded up to 64),
        if that is less than n_slots x context: the cache's pages are sized by it."""
        self.model = model
        self.rt = model.rt
        self.context = int(context)
        if self.context > model.spec.max_positions:
            raise StepError(f"context {context} exceeds the model's {model.spec.max_positions} positions")
        needs = model.cache_needs()
        want = Cache.bytes_needed(needs, n_slots, self.context, self.rt.dtype, max_tokens)
        if torch.device(self.rt.device).type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.rt.device)
            if want > free:
                raise CacheMemoryError(
                    f"the cache for {n_slots} sequences of {self.context} positions"
                    + (f" ({max_tokens} tokens in all)" if max_tokens else "") + f" needs "
                    f"{want / 2**30:.1f} GiB; {free / 2**30:.1f} GiB are free on {self.rt.device}: "
                    f"ask for fewer sequences (max_batch), a shorter context (max_context) or "
                    f"fewer tokens in all (max_tokens)")
        self.cache = Cache(needs, n_slots, self.context, self.rt.dtype, self.rt.device, max_tokens)
        self.vocab = model.spec.vocab_size
        self._graphs: "OrderedDict[tuple, dict]" = OrderedDict()    # least recently used first
        self._graph_seen: Dict[tuple, int] = {}
        self._sampling = None                 # (temperature, seed) now on the device
        self._dec: Optional[dict] = None
        self.use_graphs = True

    # -- slots -----------------------------------------------------------------
    def acquire(self, n: int) -> List[int]:
        return self.cache.acquire(n)

    def release(self, slots: Sequence[int]) -> None:
        self.cache.release(slots)

    # -- the step --------------------------------------------------------------
    def step(self, token_lists: Sequence[Sequence[int]], slots: Sequence[int],
             want: Sequence[Sequence[int]]) -> Optional[torch.Tensor]:
        """Runs ``token_lists[b]`` as the next tokens of the sequence in
        ``slots[b]``; returns float32 logits [sum(len(want[b])), vocab] in the
        order of the sequences and of ``want`` (None if nothing is wanted)."""
        if not (len(token_lists) == len(slots) == len(want)):
            raise StepError("token_lists, slots and want must have one entry per sequence")
        if len(set(slots)) != len(slots):
            raise StepError(f"a slot appears twice in one step: {list(slots)}")
        held = set(self.cache.slots.held)
        past = []
        for b, (toks, s) in enumerate(zip(token_lists, slots)):
            if s not in held:
                raise StepError(f"slot {s} is not held by a live sequence")
            if len(toks) == 0:
                raise StepError(f"sequence {b} brings no tokens")
            if self.cache.host_pos[s] + len(toks) > self.context:
                raise StepError(
                    f"sequence {b} would reach {self.cache.host_pos[s] + len(toks)} positions; "
                    f"the context is {self.context}")
            ids = np.asarray(toks, dtype=np.int64)
            if ids.ndim != 1 or int(ids.min()) < 0 or int(ids.max()) >= self.vocab:
                bad = next((t for t in toks if not 0 <= int(t) < self.vocab), toks[0])
                raise StepError(f"sequence {b}: token {bad} is outside the vocabulary "
                                f"(0..{self.vocab - 1})")
            past.append(self.cache.host_pos[s])
        try:
            self.cache.ensure(slots, [p + len(t) for p, t in zip(past, token_lists)])
        except CacheFull as e:
            raise StepError(str(e)) from None
        self.cache.sync_tables()
        batch = build_batch(token_lists, slots, past, want, self.rt.device)
        logits = self.model.forward(batch, self.cache, batch.want_rows, batch.n_want)
        ops.advance(batch, self.cache.slot_pos)
        for s, toks in zip(slots, token_lists):
            self.cache.host_pos[s] += len(toks)
        self.rt.check_status()
        return logits

    # -- decode steps that stay on the device ----------------------------------
    def _decode_buffers(self) -> dict:
        if self._dec is None:
            n = self.cache.n_slots
            dev = self.rt.device
            self._dec = {
                "tokens": torch.zeros(n, dtype=torch.int32, device=dev),
                "seq_slot": torch.zeros(n, dtype=torch.int32, device=dev),
                "row_key": torch.zeros(n, dtype=torch.int32, device=dev),
                "arange": torch.arange(n + 1, dtype=torch.int32, device=dev),
                "logits": torch.empty((n, self.vocab), dtype=torch.float32, device=dev),
                "sample_params": torch.zeros(2, dtype=torch.int64, device=dev),
                "host_params": torch.zeros(2, dtype=torch.int64).pin_memory(),
                "host": torch.zeros(3 * n, dtype=torch.int32).pin_memory(),
                "host_out": torch.zeros(n, dtype=torch.int32).pin_memory(),
            }
            # views and addresses for the per-step copies (no tensor operations on that path)
            self._dec["host_np"] = self._dec["host"].numpy()
            self._dec["host_out_np"] = self._dec["host_out"].numpy()
            self._dec["ptr"] = {k: self._dec[k].data_ptr()
                                for k in ("tokens", "seq_slot", "row_key", "host", "host_out",
                                          "sample_params", "host_params")}
        return self._dec

    def set_decode_batch(self, tokens: Sequence[int], slots: Sequence[int],
                         keys: Sequence[int]) -> None:
        """Puts the next tokens, slots and request keys of the decoding
        sequences on the device (one copy from pinned memory)."""
        d = self._decode_buffers()
        B = len(tokens)
        n = self.cache.n_slots
        h, ptr = d["host_np"], d["ptr"]
        h[0:B] = tokens
        h[n:n + B] = slots
        h[2 * n:2 * n + B] = keys
        ops.copy_async(ptr["tokens"], ptr["host"], 4 * B, True)
        ops.copy_async(ptr["seq_slot"], ptr["host"] + 4 * n, 4 * B, True)
        ops.copy_async(ptr["row_key"], ptr["host"] + 8 * n, 4 * B, True)
        d["slots_host"] = list(slots)

    def set_decode_tokens(self, tokens: Sequence[int]) -> None:
        """Only the next tokens (the decoding sequences are unchanged)."""
        d = self._decode_buffers()
        B = len(tokens)
        d["host_np"][0:B] = tokens
        ops.copy_async(d["ptr"]["tokens"], d["ptr"]["host"], 4 * B, True)

    def _decode_batch(self, B: int) -> StepBatch:
        d = self._decode_buffers()
        slots = d["slots_host"]
        past = [self.cache.host_pos[s] for s in slots]
        return StepBatch(n_tokens=B, n_seqs=B, q_lens=[1] * B, slots=list(slots), past=past,
                         tokens=d["tokens"][:B], token_seq=d["arange"][:B],
                         q_start=d["arange"][:B + 1], seq_slot=d["seq_slot"][:B],
                         want_rows=d["arange"][:B], n_want=B, ctx_bound=self._ctx_bucket(past))

    CTX_BUCKET = 512
    GRAPH_AFTER = 3       # a decode shape is captured on its third step
    MAX_GRAPHS = 16       # captured decode shapes kept (the least recently used goes first)

    def _set_sampling(self, temperature: float, seed: int) -> None:
        """Seed and temperature live on the device, where the sampling kernel reads them:
        a captured step serves every seed and temperature."""
        if self._sampling == (temperature, seed):
            return
        d = self._decode_buffers()
        d["host_params"][0], d["host_params"][1] = sampling.device_params(temperature, seed)
        ops.copy_async(d["ptr"]["sample_params"], d["ptr"]["host_params"], 16, True)
        ops.stream_wait()                     # the pinned words may change again right away
        self._sampling = (temperature, seed)

    def _ctx_bucket(self, past: Sequence[int]) -> int:
        """The longest sequence after this step, rounded up: launches sized by it
        stay valid (and a captured graph reusable) until a sequence crosses it."""
        longest = max(past) + 1
        return min(self.context, -(-longest // self.CTX_BUCKET) * self.CTX_BUCKET)

    def _decode_body(self, B: int) -> None:
        d = self._decode_buffers()
        batch = self._decode_batch(B)
        logits = self.model.forward(batch, self.cache, batch.want_rows, B, logits_out=d["logits"][:B])
        ops.advance(batch, self.cache.slot_pos)
        # the new token goes where the next step's embedding reads it
        sampling.sample(logits, 0.0, 0, d["row_key"][:B], batch.seq_slot, self.cache.slot_pos,
                   d["tokens"][:B], params=d["sample_params"])

    def decode_step(self, B: int, temperature: float, seed: int) -> None:
        """One decode step of the B sequences set by ``set_decode_batch``: their
        tokens are read from, and their sampled successors written to, the
        device token buffer.  Nothing crosses to the host."""
        d = self._decode_buffers()
        live = d["slots_host"][:B]
        for s in live:
            if self.cache.host_pos[s] + 1 > self.context:
                raise StepError(f"the sequence in slot {s} is at the context's end ({self.context})")
        try:
            self.cache.ensure(live, [self.cache.host_pos[s] + 1 for s in live])
        except CacheFull as e:
            raise StepError(str(e)) from None
        self.cache.sync_tables()
        self._set_sampling(float(temperature), int(seed))
        if not self.use_graphs:
            self._decode_body(B)
        else:
            key = (B, self._ctx_bucket([self.cache.host_pos[s] for s in d["slots_host"][:B]]))
            g = self._graphs.get(key)
            if g is not None and g["generation"] != self.rt.buffer_generation:
                del self._graphs[key]         # a scratch buffer moved since the capture
                g = None
            seen = self._graph_seen.get(key, 0) + 1
            self._graph_seen[key] = seen
            if g is None and seen < self.GRAPH_AFTER:
                # a shape that may not last (a batch that is shrinking step by step): not
                # worth a capture yet
                self._decode_body(B)
            elif g is None:
                # this step runs eagerly once more (every scratch buffer has its final
                # size); then the same launches are captured for replays
                self._decode_body(B)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                self.rt.frozen = True
                before = ops.LAUNCHES
                try:
                    with torch.cuda.graph(graph):
                        self._decode_body(B)
                finally:
                    self.rt.frozen = False
                captured = ops.LAUNCHES - before
                ops.LAUNCHES = before             # capturing launches nothing
                self._graphs[key] = {"graph": graph, "generation": self.rt.buffer_generation,
                                     "kernels": captured}
                while len(self._graphs) > self.MAX_GRAPHS:
                    old, _ = self._graphs.popitem(last=False)
                    self._graph_seen.pop(old, None)
            else:
                self._graphs.move_to_end(key)
                g["graph"].replay()
                ops.LAUNCHES += g["kernels"]
        for s in d["slots_host"][:B]:
            self.cache.host_pos[s] += 1

    def read_decode_tokens(self, B: int) -> List[int]:
        d = self._decode_buffers()
        ops.copy_async(d["ptr"]["host_out"], d["ptr"]["tokens"], 4 * B, False)
        ops.stream_wait()
        return d["host_out_np"][:B].tolist()

    def decode_logits(self, B: int) -> torch.Tensor:
        return self._decode_buffers()["logits"][:B]
