"""The cache: per-sequence slots, keys and values per layer run, each
sequence's own length, and fixed-size per-sequence state beside them.

What a mixer needs is declared by the mixer (one ``CacheNeed``, or several by
name: keys and values AND a state, two states of different types); needs that are
equal share one *group*, which has storage of its own:

* ``kv`` groups hold keys and values.  A sequence's rows are numbered
  0 .. capacity - 1; ``capacity`` is the window when the mixer has one (the rows are
  then a ring: position p lives at row p % capacity), else the context length.
  When the tokens that live sequences hold together are bounded (``max_tokens``)
  the rows live in pages of ``PAGE`` = 64 positions,
  ``K, V : [entries, kv_heads, pages, PAGE, head_dim]``, with a table
  ``[slots, pages_per_slot]`` that names the page of rows 64 p .. 64 p + 63 of each
  sequence: a sequence takes a page from the group's pool when it grows into it and
  gives all back when it ends, so the memory follows the tokens that are held, not
  slots x capacity.  Without such a bound every slot can fill up anyway, and each
  sequence has one block of its own, ``K, V : [entries, slots, kv_heads, capacity,
  head_dim]``, no table: the decode attention streams from that layout 5 to 20 %
  faster (batch 8 to 64 at 7B sizes).
* ``state`` groups hold ``[entries, slots, *shape]`` of fixed size per
  sequence; it is zeroed when a slot is acquired.  The Llama / Mistral decoder
  declares none; the storage exists for mixers that carry a recurrent state.

The per-sequence record on the device is ``slot_pos[slot]``: the number of
positions the sequence has taken so far (its next position).  Ring offset and
valid length follow from it (pos % capacity, min(pos, capacity)).  Kernels read
it, and the page table, on the device, so a captured decode step needs no new
arguments per step.  The reference keeps one sequence's cache inside each block,
f16[S, G*hd] (model.h:241-243, model.cpp:201-202) and passes kv_pos/kv_len per call
(infer.cpp:486-488).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .slots import SlotAllocator, SlotError

PAGE = 64      # positions per page (the kernels' KV_PAGE)


class CacheFull(SlotError):
    """The pool of pages cannot hold the tokens that were asked for."""


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
    k: Optional[torch.Tensor] = None           # [kv_heads, pages, PAGE, head_dim], or without
    v: Optional[torch.Tensor] = None           # pages [slots, kv_heads, capacity, head_dim]
    pages: Optional[torch.Tensor] = None       # int32 [slots, pages_per_slot] on the device, or None
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


def _pool_pages(need: CacheNeed, n_slots: int, context: int, max_tokens: Optional[int]) -> int:
    """Pages in a kv group's pool when the tokens that live sequences hold together are
    bounded (each count rounded up to a page); 0 when every slot can fill up anyway and
    the group keeps one block per sequence instead."""
    per_slot = -(-need.capacity(context) // PAGE)
    full = n_slots * per_slot
    if max_tokens is None or -(-int(max_tokens) // PAGE) >= full:
        return 0
    return max(1, -(-int(max_tokens) // PAGE))


class Cache:
    def __init__(self, needs: Dict[object, CacheNeed], n_slots: int, context: int,
                 dtype: torch.dtype, device, max_tokens: Optional[int] = None):
        """``needs`` maps a key to a need.  The model's keys are (run entry, mixer
        name, need name); any hashable, sortable key will do (entries that read
        another entry's cache are absent).  ``context`` is the most positions one
        sequence may take; ``max_tokens``, if given, the most tokens all live sequences
        hold together (each sequence's count rounded up to a multiple of 64): it sizes
        the page pools."""
        self.n_slots = n_slots
        self.context = context
        self.dtype = dtype
        self.device = torch.device(device)
        self.on_gpu = self.device.type == "cuda"
        self.slots = SlotAllocator(n_slots)
        self.slot_pos = torch.zeros(n_slots, dtype=torch.int32, device=self.device)
        self.host_pos = [0] * n_slots          # the host's copy of slot_pos
        self._covered = [0] * n_slots          # positions each slot can hold with the pages it has
        self._paged = False                    # whether any group keeps its rows in pages
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
                n_pages = _pool_pages(need, n_slots, context, max_tokens)
                g["capacity"] = cap
                if n_pages == 0:                                   # one block per sequence
                    shape = (n, n_slots, need.kv_heads, cap, need.head_dim)
                    g["k"] = torch.zeros(shape, dtype=dtype, device=self.device)
                    g["v"] = torch.zeros(shape, dtype=dtype, device=self.device)
                    continue
                shape = (n, need.kv_heads, n_pages, PAGE, need.head_dim)
                g["pages_per_slot"] = -(-cap // PAGE)
                g["k"] = torch.zeros(shape, dtype=dtype, device=self.device)
                g["v"] = torch.zeros(shape, dtype=dtype, device=self.device)
                g["pool"] = SlotAllocator(n_pages, what="page")
                g["held"] = [[] for _ in range(n_slots)]           # a slot's pages, in row order
                table = torch.zeros((n_slots, g["pages_per_slot"]), dtype=torch.int32)
                g["table_host"] = table.pin_memory() if self.on_gpu else table
                g["table"] = torch.zeros_like(table, device=self.device)
                g["dirty"] = set()                                 # slots whose row must go down
                self._paged = True
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
                     dtype: torch.dtype, max_tokens: Optional[int] = None) -> int:
        esz = torch.empty((), dtype=dtype).element_size()
        total = 0
        for need in needs.values():
            if need.kind == "kv":
                pages = _pool_pages(need, n_slots, context, max_tokens)
                rows = pages * PAGE if pages else n_slots * need.capacity(context)
                total += 2 * rows * need.kv_heads * need.head_dim * esz
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
        """Gives the slots and their pages back.  Work that is still queued on the
        device for these sequences ends first: their pages may be handed out at once."""
        slots = list(slots)
        self.slots.release(slots)
        if self.on_gpu:
            torch.cuda.current_stream(self.device).synchronize()
        for g in self.groups:
            if "pool" in g:
                for s in slots:
                    if g["held"][s]:
                        g["pool"].release(g["held"][s])
                        g["held"][s] = []
        for s in slots:
            self._covered[s] = 0

    # -- pages ---------------------------------------------------------------
    def free_pages(self) -> List[int]:
        """Free pages of each kv group, in group order."""
        return [g["pool"].free_count for g in self.groups if "pool" in g]

    def ensure(self, slots: Sequence[int], lengths: Sequence[int]) -> None:
        """Pages for the sequences in ``slots`` to hold ``lengths`` positions.  Either
        all of them are found or nothing changes and ``CacheFull`` is raised."""
        if not self._paged or all(n <= self._covered[s] for s, n in zip(slots, lengths)):
            return                              # no pages, or the usual case of a decode step
        plan = []
        for g in self.groups:
            if "pool" not in g:
                continue
            want = []
            for s, n in zip(slots, lengths):
                need = -(-min(int(n), g["capacity"]) // PAGE) - len(g["held"][s])
                if need > 0:
                    want.append((s, need))
            total = sum(n for _, n in want)
            if total > g["pool"].free_count:
                raise CacheFull(
                    f"{total} more pages of {PAGE} positions are needed and {g['pool'].free_count} of "
                    f"{g['pool'].n_slots} are free: the live sequences hold more tokens than the "
                    f"cache was sized for (max_tokens / max_batch x max_context)")
            plan.append((g, want))
        for g, want in plan:
            for s, n in want:
                pages = g["pool"].acquire(n)
                at = len(g["held"][s])
                g["held"][s].extend(pages)
                g["table_host"][s, at:at + n] = torch.tensor(pages, dtype=torch.int32)
                g["dirty"].add(s)
        for s in slots:
            self._covered[s] = min([self.context] + [
                len(g["held"][s]) * PAGE for g in self.groups
                if "pool" in g and len(g["held"][s]) < g["pages_per_slot"]])

    def sync_tables(self) -> None:
        """The changed rows of the page tables go to the device, in stream order before
        the kernels that read them."""
        for g in self.groups:
            if "pool" not in g or not g["dirty"]:
                continue
            if self.on_gpu:
                from ..csrc import ops
                row = g["pages_per_slot"] * 4
                for s in sorted(g["dirty"]):
                    ops.copy_async(g["table"].data_ptr() + s * row, g["table_host"].data_ptr() + s * row,
                                   row, True)
            else:
                g["table"].copy_(g["table_host"])
            g["dirty"].clear()

    # -- views ---------------------------------------------------------------
    def view(self, entry) -> CacheView:
        if entry not in self._entry:
            raise KeyError(f"{entry!r} owns no cache")
        gi, i = self._entry[entry]
        g = self.groups[gi]
        if g["need"].kind == "kv":
            return CacheView("kv", capacity=g["capacity"], k=g["k"][i], v=g["v"][i],
                             slot_pos=self.slot_pos, pages=g.get("table"))
        return CacheView("state", state=g["state"][i], slot_pos=self.slot_pos)

    def rows(self, entry, slot: int, first: int = 0, count: Optional[int] = None):
        """Keys and values of rows ``first .. first + count - 1`` of the sequence in
        ``slot`` as two tensors [kv_heads, count, head_dim] (a gather through the page
        table, for inspection and tests)."""
        gi, i = self._entry[entry]
        g = self.groups[gi]
        if "pool" not in g:
            count = g["capacity"] - first if count is None else count
            return g["k"][i][slot][:, first:first + count], g["v"][i][slot][:, first:first + count]
        held = g["held"][slot]
        count = len(held) * PAGE - first if count is None else count
        idx = torch.tensor([held[r // PAGE] * PAGE + r % PAGE for r in range(first, first + count)],
                           dtype=torch.long, device=self.device)
        flat = lambda t: t[i].reshape(t.shape[1], -1, t.shape[4])
        return flat(g["k"])[:, idx], flat(g["v"])[:, idx]

    def room(self, slot: int) -> int:
        """Positions the sequence in ``slot`` may still take."""
        return self.context - self.host_pos[slot]
