"""The cache: per-sequence slots, keys and values per layer run, each
sequence's own length, and fixed-size per-sequence state beside them.

What a mixer needs is declared by the mixer (one ``CacheNeed``, or several by
name: keys and values AND a state, two states of different types); needs that are
equal share one *group*, which has storage of its own:

* ``kv`` groups hold ``K, V : [entries, slots, kv_heads, capacity, head_dim]``.
  ``capacity`` is the window when the mixer has one (the slot is then a ring:
  position p lives at row p % capacity), else the context length.
* ``state`` groups hold ``[entries, slots, *shape]`` of fixed size per
  sequence; it is zeroed when a slot is acquired.  The Llama / Mistral decoder
  declares none; the storage exists for mixers that carry a recurrent state.

The per-sequence record on the device is ``slot_pos[slot]``: the number of
positions the sequence has taken so far (its next position).  Ring offset and
valid length follow from it (pos % capacity, min(pos, capacity)).  Kernels read
it on the device, so a captured decode step needs no new arguments per step.
The reference keeps one sequence's cache inside each block, f16[S, G*hd]
(model.h:241-243, model.cpp:201-202) and passes kv_pos/kv_len per call
(infer.cpp:486-488).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .slots import SlotAllocator


@dataclass(frozen=True)
class CacheNeed:
    """What one run entry's mixer asks of the cache."""
    kind: str                                  # "kv" or "state"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None               # kv: keep only the last `window` positions
    state_shape: Tuple[int, ...] = ()          # state: per-sequence shape
    state_dtype: torch.dtype = torch.float32

    def group_key(self, context: int):
        if self.kind == "kv":
            return ("kv", self.kv_heads, self.head_dim, self.capacity(context))
        return ("state", tuple(self.state_shape), self.state_dtype)

    def capacity(self, context: int) -> int:
        return context if self.window is None else min(context, self.window)


@dataclass
class CacheView:
    """What a mixer sees of the cache for one run entry."""
    kind: str
    capacity: int = 0
    k: Optional[torch.Tensor] = None           # [slots, kv_heads, capacity, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None       # [slots, *shape]
    slot_pos: Optional[torch.Tensor] = None    # int32 [slots]
    kv_step: Optional[torch.Tensor] = None     # this step's keys/values, kept for a reader entry


def normalise_needs(need) -> Dict[str, CacheNeed]:
    """What a mixer's ``cache_need()`` may return -- nothing, one need, or several by
    name -- as a dict.  A single need goes by the name "cache"."""
    if need is None:
        return {}
    if isinstance(need, CacheNeed):
        return {"cache": need}
    out = dict(need)
    for name, n in out.items():
        if not isinstance(n, CacheNeed):
            raise TypeError(f"cache need {name!r} is a {type(n).__name__}, not a CacheNeed")
    return out


class Cache:
    def __init__(self, needs: Dict[object, CacheNeed], n_slots: int, context: int,
                 dtype: torch.dtype, device):
        """``needs`` maps a key to a need.  The model's keys are (run entry, mixer
        name, need name); any hashable, sortable key will do (entries that read
        another entry's cache are absent).  ``context`` is the most positions one
        sequence may take."""
        self.n_slots = n_slots
        self.context = context
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = SlotAllocator(n_slots)
        self.slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=self.device)
        self.host_pos = [0] * n_slots          # the host's copy of slot_pos
        self.groups: List[dict] = []
        self._entry: Dict[object, Tuple[int, int]] = {}
        by_key: Dict[tuple, int] = {}
        for entry in sorted(needs):
            need = needs[entry]
            key = need.group_key(context)
            if key not in by_key:
                by_key[key] = len(self.groups)
                self.groups.append({"key": key, "need": need, "entries": []})
            g = by_key[key]
            self._entry[entry] = (g, len(self.groups[g]["entries"]))
            self.groups[g]["entries"].append(entry)
        for g in self.groups:
            need, n = g["need"], len(g["entries"])
            if need.kind == "kv":
                cap = need.capacity(context)
                shape = (n, n_slots, need.kv_heads, cap, need.head_dim)
                g["capacity"] = cap
                g["k"] = torch.zeros(shape, dtype=dtype, device=self.device)
                g["v"] = torch.zeros(shape, dtype=dtype, device=self.device)
            elif need.kind == "state":
                g["state"] = torch.zeros((n, n_slots) + tuple(need.state_shape),
                                         dtype=need.state_dtype, device=self.device)
            else:
                raise ValueError(f"unknown cache kind {need.kind!r}")

    # -- sizes ---------------------------------------------------------------
    def bytes(self) -> int:
        total = 0
        for g in self.groups:
            for name in ("k", "v", "state"):
                if name in g:
                    total += g[name].numel() * g[name].element_size()
        return total

    @staticmethod
    def bytes_needed(needs: Dict[object, CacheNeed], n_slots: int, context: int,
                     dtype: torch.dtype) -> int:
        esz = torch.empty((), dtype=dtype).element_size()
        total = 0
        for need in needs.values():
            if need.kind == "kv":
                total += 2 * n_slots * need.kv_heads * need.capacity(context) * need.head_dim * esz
            else:
                n = 1
                for s in need.state_shape:
                    n *= s
                total += n_slots * n * torch.empty((), dtype=need.state_dtype).element_size()
        return total

    # -- slots ---------------------------------------------------------------
    def acquire(self, n: int) -> List[int]:
        slots = self.slots.acquire(n)
        idx = torch.tensor(slots, dtype=torch.long, device=self.device)
        self.slot_pos.index_fill_(0, idx, 0)
        for g in self.groups:
            if "state" in g:
                g["state"].index_fill_(1, idx, 0)
        for s in slots:
            self.host_pos[s] = 0
        return slots

    def release(self, slots: Sequence[int]) -> None:
        self.slots.release(slots)

    # -- views ---------------------------------------------------------------
    def view(self, entry) -> CacheView:
        if entry not in self._entry:
            raise KeyError(f"{entry!r} owns no cache")
        gi, i = self._entry[entry]
        g = self.groups[gi]
        if g["need"].kind == "kv":
            return CacheView("kv", capacity=g["capacity"], k=g["k"][i], v=g["v"][i],
                             slot_pos=self.slot_pos)
        return CacheView("state", state=g["state"][i], slot_pos=self.slot_pos)

    def room(self, slot: int) -> int:
        """Positions the sequence in ``slot`` may still take."""
        return self.context - self.host_pos[slot]
