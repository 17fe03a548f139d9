"""The Python entry point: a model folder (or a configuration and a seed) in,
logits or generated tokens out.

    lm = LM.from_pretrained("model_dir", dtype="bfloat16", max_context=4096, max_batch=8)
    out = lm.generate([[1, 5, 9], [1, 7]], max_new_tokens=32, temperature=0.0)
    out[0].tokens, out[0].finish_reason

The reference has no Python interface; its C++ ``main`` is the counterpart
(main.cpp:54-148), mirrored by ``python -m yalm_b200``.
"""
from __future__ import annotations

import math
import os
import time
from typing import Any, Dict, List, Optional, Sequence, Union

import torch

from ..config import config_from_dict, load_config
from .. import sampling
from ..csrc import ops
from ..parts import Model, Runtime
from ..weights import load_checkpoint, load_packed, random_tensors, write_model_dir
from .generate import Completion, run_generation
from .step import Engine

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float16": torch.float16,
           "fp16": torch.float16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float16: torch.float16,
           torch.float32: torch.float32}


def _dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype must be 'bfloat16', 'float16' or 'float32', got {d!r}")
    return _DTYPES[d]


class LM:
    def __init__(self, config: Any, tensors: Dict[str, torch.Tensor], dtype="bfloat16",
                 max_context: Optional[int] = None, max_batch: int = 8, device="cuda:0",
                 gemm: str = "auto", attention: str = "auto", float32_matrices: str = "keep",
                 window_override: Optional[int] = None, max_tokens: Optional[int] = None):
        """``max_context``: the most positions a sequence may take (at most the model's).
        ``max_tokens``: the most tokens all live sequences hold together (each count
        rounded up to 64), when that is less than max_batch x max_context: the cache's
        pages are sized by it.
        ``window_override=n``: attention parts without a window (or with a longer one)
        see only the last n positions, so the cache is a ring of n rows per sequence
        and generation goes on past n: the role of the reference's ``-T n``
        (model.cpp:28-32), as a pure window."""
        if window_override:
            if not hasattr(config, "with_window"):
                raise ValueError(f"{type(config).__name__} has no window to impose")
            config = config.with_window(int(window_override))
        self.config = config
        self.spec = config.to_spec()
        self.rt = Runtime(_dtype(dtype), device, gemm=gemm, attention=attention,
                          float32_matrices=float32_matrices)
        self.model = Model(self.spec, self.rt)
        ignorable = getattr(config, "ignorable_tensor", None)
        self.model.bind(tensors, ignore_unexpected=[n for n in tensors if ignorable(n)] if ignorable else ())
        context = self.spec.max_positions if not max_context else min(int(max_context),
                                                                     self.spec.max_positions)
        self.engine = Engine(self.model, max_batch, context, max_tokens)
        self._next_key = 0

    # -- construction ----------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir: str, **kw) -> "LM":
        """A model folder (config.json and safetensors files), or one packed file
        (``python -m yalm_b200.weights.pack``) with the configuration in its metadata."""
        if os.path.isfile(model_dir):
            config, tensors = load_packed(model_dir)
            return cls(config_from_dict(config), tensors, **kw)
        config = load_config(model_dir)
        return cls(config, load_checkpoint(model_dir), **kw)

    @classmethod
    def from_random(cls, config: Union[dict, Any], seed: int = 0, dtype="bfloat16",
                    std: float = 0.02, norm_jitter: float = 0.02, device="cuda:0", **kw) -> "LM":
        """Random weights drawn on the device (no model folder is written)."""
        if isinstance(config, dict):
            config = config_from_dict(config)
        dt = _dtype(dtype)
        tensors = random_tensors(tensor_needs_of(config), seed, dtype=dt, std=std,
                                 norm_jitter=norm_jitter, device=device)
        return cls(config, tensors, dtype=dtype, device=device, **kw)

    @staticmethod
    def write_random_model(out_dir: str, config: Union[dict, Any], seed: int = 0,
                           dtype="bfloat16", std: float = 0.02, norm_jitter: float = 0.02) -> None:
        """Random-weights mode: writes config.json and model.safetensors."""
        if isinstance(config, dict):
            config = config_from_dict(config)
        write_model_dir(out_dir, config, tensor_needs_of(config), seed, dtype=_dtype(dtype),
                        std=std, norm_jitter=norm_jitter)

    # -- the step function -----------------------------------------------------
    @property
    def context(self) -> int:
        return self.engine.context

    @property
    def max_batch(self) -> int:
        return self.engine.cache.n_slots

    def acquire(self, n: int) -> List[int]:
        return self.engine.acquire(n)

    def release(self, slots: Sequence[int]) -> None:
        self.engine.release(slots)

    def step(self, token_lists, slots, want) -> Optional[torch.Tensor]:
        return self.engine.step(token_lists, slots, want)

    # -- generation ------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256,
                 temperature: float = 1.0, seed: int = 0, stop_ids: Optional[Sequence[int]] = None,
                 ignore_eos: bool = False, on_token=None) -> List[Completion]:
        """Continues every prompt.  ``temperature == 0`` is greedy.  Stop tokens
        default to the configuration's eos ids; the stop token is part of the
        output.  Requests beyond ``max_batch`` run as further batches."""
        if stop_ids is None:
            stop_ids = [] if ignore_eos else list(self.spec.stop_token_ids)
        backend = _DeviceBackend(self, float(temperature), int(seed))
        t0 = time.perf_counter()
        out = run_generation(backend, prompts, max_new_tokens, stop_ids, on_token=on_token)
        self.rt.check_status()
        self.last_stats = {"seconds": time.perf_counter() - t0,
                           "prefill_seconds": backend.prefill_seconds,
                           "prompt_tokens": sum(len(p) for p in prompts),
                           "new_tokens": sum(len(c.tokens) for c in out),
                           "decode_steps": backend.decode_steps,
                           "decode_seconds": backend.decode_seconds,
                           "step_seconds": backend.step_seconds,
                           "h2d_bytes": backend.h2d_bytes, "d2h_bytes": backend.d2h_bytes}
        return out

    def perplexity(self, tokens: Sequence[int], chunk: int = 2048):
        """exp(-mean log p(next token)) over one text and its error estimate, as the
        reference's perplexity mode (main.cpp:150-235), which walks a text of any length."""
        tokens = list(tokens)
        if len(tokens) < 2:
            raise ValueError("perplexity needs at least two tokens")
        # The text runs through the step function in portions of at most `chunk` tokens
        # (that bounds the logits held at once).  A text longer than the context is cut
        # into sequences of `context` tokens that overlap by one token, so that every
        # token but the first is predicted exactly once; each starts from an empty cache.
        C = self.context
        s = ss = 0.0
        n = 0
        start = 0
        while start < len(tokens) - 1:
            seg = tokens[start:start + C]
            slot = self.acquire(1)
            try:
                for a in range(0, len(seg) - 1, chunk):
                    b = min(len(seg) - 1, a + chunk)
                    logits = self.step([seg[a:b]], slot, [list(range(b - a))])
                    lp = torch.log_softmax(logits.double(), -1)
                    nxt = torch.tensor(seg[a + 1:b + 1], device=lp.device)
                    vals = lp.gather(1, nxt[:, None])[:, 0]
                    s += vals.sum().item()
                    ss += (vals * vals).sum().item()
                    n += vals.numel()
            finally:
                self.release(slot)
            start += len(seg) - 1
        ppl = math.exp(-s / n)
        return ppl, ppl * math.sqrt(max(0.0, (ss - s * s / n) / n / n))


def tensor_needs_of(config) -> dict:
    """The tensors a configuration's model declares (no device needed)."""
    return Model(config.to_spec(), Runtime.shapes_only()).tensor_needs()


class _DeviceBackend:
    """The generation loop's view of the engine (see generate.py)."""

    def __init__(self, lm: LM, temperature: float, seed: int):
        self.lm = lm
        self.engine = lm.engine
        self.temperature = temperature
        self.seed = seed
        self.max_batch = lm.max_batch
        self.context = lm.context
        self.prefill_seconds = 0.0
        self.decode_seconds = 0.0
        self.step_seconds = []                # wall time of each decode step, host to host
        self.decode_steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def begin(self, prompts, keys):
        """Prefill and first tokens.  The batch's rows sit on the device in the order the
        model's mixers ask for (the attention part: longest sequence first); `rank` maps
        the caller's order to that one.  All sequences grow alike, so the order holds for
        the batch's life."""
        eng = self.engine
        B = len(prompts)
        order = self.lm.model.row_order([len(p) for p in prompts])
        slots = eng.acquire(B)
        try:
            t0 = time.perf_counter()
            rows = [prompts[i] for i in order]
            logits = eng.step(rows, slots, [[len(p) - 1] for p in rows])
            d = eng._decode_buffers()
            # sample the first token of every sequence into the decode token buffer
            eng.set_decode_batch([0] * B, slots, [keys[i] for i in order])
            sampling.sample(logits, self.temperature, self.seed, d["row_key"][:B], d["seq_slot"][:B],
                       eng.cache.slot_pos, d["tokens"][:B])
            sampled = eng.read_decode_tokens(B)
            self.prefill_seconds += time.perf_counter() - t0
        except Exception:
            eng.release(slots)
            raise
        rank = [0] * B
        for r, i in enumerate(order):
            rank[i] = r
        first = [sampled[rank[i]] for i in range(B)]
        handle = {"slots": slots, "keys": [keys[i] for i in order], "rank": rank,
                  "active": list(range(B)), "rows": list(range(B)), "perm": order,
                  "held": set(slots)}
        return handle, first

    def decode(self, handle, active, tokens):
        """One step: the host's tokens go down (pinned memory), the sampled
        tokens come back; slots and keys go down only when the batch shrank."""
        eng = self.engine
        t0 = time.perf_counter()
        B = len(active)
        if active != handle["active"]:
            rank = handle["rank"]
            # sequences that ended give their slot and pages back now, not at the batch's end
            gone = [handle["slots"][rank[j]] for j in handle["active"] if j not in set(active)]
            eng.release(gone)
            handle["held"] -= set(gone)
            # perm[r]: which entry of `active` sits in device row r; rows[r]: its row at the start
            perm = sorted(range(B), key=lambda k: rank[active[k]])
            rows = [rank[active[k]] for k in perm]
            handle["active"], handle["perm"], handle["rows"] = list(active), perm, rows
            eng.set_decode_batch([tokens[k] for k in perm], [handle["slots"][r] for r in rows],
                                 [handle["keys"][r] for r in rows])
            self.h2d_bytes += 12 * B
        else:
            perm = handle["perm"]
            eng.set_decode_tokens([tokens[k] for k in perm])
            self.h2d_bytes += 4 * B
        eng.decode_step(B, self.temperature, self.seed)
        sampled = eng.read_decode_tokens(B)
        out = [0] * B
        for r, k in enumerate(perm):
            out[k] = sampled[r]
        self.d2h_bytes += 4 * B
        self.decode_steps += 1
        dt = time.perf_counter() - t0
        self.decode_seconds += dt
        self.step_seconds.append(dt)
        return out

    def end(self, handle):
        self.engine.release(sorted(handle["held"]))
        handle["held"] = set()
