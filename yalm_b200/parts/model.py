"""A model assembled from a :class:`ModelSpec`: embedding, the layers in their
run order, final norm, head.  It declares the tensors it needs by checkpoint
name, binds a checkpoint, declares what it needs of the cache, and runs one
step over a batch (``forward``), returning logits at the wanted rows.

The reference's counterpart is ``Model``/``Block`` (model.h:149-270,
model.cpp:356-428): weights bound by name, blocks run in order, final norm and
classifier skipped when no logits are wanted (infer.cu:1172-1176).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional

import torch

from ..cache import Cache, CacheNeed
from ..cache.storage import normalise_needs
from ..config import ModelSpec
from ..weights import TensorNeed, check_tensors
from .base import (BLOCKS, EMBEDDINGS, HEADS, NORMS, ResidualStream, Runtime, make_part)


class Model:
    def __init__(self, spec: ModelSpec, rt: Runtime):
        spec.validate()
        self.spec = spec
        self.rt = rt
        self.embedding = make_part(EMBEDDINGS, spec.embedding, rt)
        if spec.layers and spec.layers[0].block not in BLOCKS:
            raise KeyError(f"no block arrangement {spec.layers[0].block!r} is registered")
        self.layers = []
        for ls in spec.layers:
            if ls.block not in BLOCKS:
                raise KeyError(f"no block arrangement {ls.block!r} is registered")
            self.layers.append(BLOCKS[ls.block](ls, rt))
        self.final_norm = make_part(NORMS, spec.final_norm, rt)
        self.head = make_part(HEADS, spec.head, rt)
        self.run_order = list(spec.run_order)
        self._readers = {e.reads_cache_of for e in self.run_order if e.reads_cache_of is not None}
        self._last_reader = {e.reads_cache_of: i for i, e in enumerate(self.run_order)
                             if e.reads_cache_of is not None}

    # -- weights -------------------------------------------------------------
    def _bound_parts(self):
        yield self.embedding, self.spec.embedding
        for layer in self.layers:
            yield from layer.parts()
        yield self.final_norm, self.spec.final_norm
        yield self.head, self.spec.head

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        """Checkpoint name -> need, over all parts (a tensor two parts share is
        listed once and must have one shape)."""
        out: Dict[str, TensorNeed] = {}
        for part, pspec in self._bound_parts():
            for key, need in part.tensor_needs().items():
                if key not in pspec.tensors:
                    raise KeyError(f"part {pspec.kind!r} needs tensor {key!r} but the "
                                   f"architecture names no checkpoint tensor for it")
                name = pspec.tensors[key]
                if name in out and tuple(out[name].shape) != tuple(need.shape):
                    raise ValueError(f"tensor {name!r} is wanted with shapes "
                                     f"{out[name].shape} and {need.shape}")
                out.setdefault(name, need)
        return out

    def bind(self, tensors: Dict[str, torch.Tensor], ignore_unexpected=()) -> None:
        """One error lists every missing, unexpected and mis-shaped tensor."""
        check_tensors(self.tensor_needs(), tensors, optional_unexpected=tuple(ignore_unexpected))
        for part, pspec in self._bound_parts():
            part.bind({key: tensors[pspec.tensors[key]] for key in part.tensor_needs()})
        self.rt.end_binding()

    # -- cache ---------------------------------------------------------------
    def cache_needs(self) -> Dict[tuple, CacheNeed]:
        """(run entry, mixer name, need name) -> what that mixer asks of the cache.  A
        mixer may declare one need or several by name; entries that read another
        entry's cache own none."""
        needs = {}
        for i, e in enumerate(self.run_order):
            if e.reads_cache_of is not None:
                continue
            for mname, mixer in self.layers[e.layer].mixers().items():
                for nname, need in normalise_needs(mixer.cache_need()).items():
                    needs[(i, mname, nname)] = need
        return needs

    def _views_of(self, owner: int, batch, cache: Cache):
        """mixer name -> what that mixer sees of run entry ``owner``'s cache: one view,
        a dict of views by need name, or None."""
        rt = self.rt
        out = {}
        for mname, mixer in self.layers[self.run_order[owner].layer].mixers().items():
            needs = normalise_needs(mixer.cache_need())
            got = {}
            for nname, need in needs.items():
                view = cache.view((owner, mname, nname))
                if view.kind == "kv" and owner in self._readers:
                    # this step's keys and values are kept apart for the entries that read them
                    view = dataclasses.replace(view, kv_step=rt.buffer(
                        f"kv_step_{owner}_{mname}_{nname}",
                        (batch.n_tokens, 2, need.kv_heads, need.head_dim), rt.dtype))
                got[nname] = view
            out[mname] = None if not got else (got["cache"] if list(got) == ["cache"] else got)
        return out

    # -- what a step costs (for roofline figures) ------------------------------
    def step_bytes(self, contexts) -> int:
        """Bytes a decode step of sequences with these context lengths has to read:
        every weight once (of the embedding table one row per sequence) and the cache
        of the live sequences."""
        esz = torch.empty((), dtype=self.rt.dtype).element_size()
        needs = self.tensor_needs()                  # declared shapes: no device needed
        table_name = self.spec.embedding.tensors.get("weight")
        tied = table_name in self.spec.head.tensors.values()
        total = 0
        for name, need in needs.items():
            n = 1
            for d in need.shape:
                n *= int(d)
            if name == table_name and not tied:
                n = len(contexts) * int(need.shape[-1])      # an untied table is read by rows only
            elif name == table_name:
                n += len(contexts) * int(need.shape[-1])
            total += n * (4 if need.init == "ones" else esz)
        for e in self.run_order:
            for mixer in self.layers[e.layer].mixers().values():
                f = getattr(mixer, "cache_read_bytes", None)
                if f is not None:
                    total += f(contexts, esz)
        return total

    def step_flops(self, q_lens, past=None, n_want: int = 1) -> float:
        """Floating-point operations of one step (products and attention)."""
        past = [0] * len(q_lens) if past is None else list(past)
        total = 0.0
        for e in self.run_order:
            for part, _ in self.layers[e.layer].parts():
                f = getattr(part, "flops", None)
                if f is not None:
                    total += f(q_lens, past)
        f = getattr(self.head, "flops", None)
        return total + (f([n_want], [0]) if f is not None else 0.0)

    def row_order(self, lengths) -> list:
        """The order in which a batch's sequences should sit in the step's rows: longest
        first if a mixer asks for it (``prefers_longest_first``), else as given."""
        idx = list(range(len(lengths)))
        if any(getattr(m, "prefers_longest_first", False)
               for layer in self.layers for m in layer.mixers().values()):
            idx.sort(key=lambda i: -lengths[i])
        return idx

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part, _ in self._bound_parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    # -- one step --------------------------------------------------------------
    def forward(self, batch, cache: Cache, want_rows: Optional[torch.Tensor], n_want: int,
                logits_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the batch's tokens through every run entry, writing the cache;
        returns float32 logits [n_want, vocab] (None when nothing is wanted).
        Positions are NOT advanced here (the step function does that)."""
        rt = self.rt
        x = self.embedding.forward(batch)
        stream = ResidualStream(rt, x)
        views = {}
        deferred: Dict[int, list] = {}      # run entry -> cache writes to make once it has run
        for i, e in enumerate(self.run_order):
            layer = self.layers[e.layer]
            owner = i if e.reads_cache_of is None else e.reads_cache_of
            if owner not in views:
                views[owner] = self._views_of(owner, batch, cache)
            later = layer.forward(stream, batch, views[owner], shared=e.reads_cache_of is not None)
            if later is not None:
                # a write the mixer may only make after every entry that reads its cache
                deferred.setdefault(self._last_reader.get(i, i), []).append(later)
            for write in deferred.pop(i, []):
                write()
        if n_want == 0:
            return None
        h = self.final_norm(stream, rows=want_rows, n_rows=n_want, name="final_normed")
        if logits_out is None:
            logits_out = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32,
                                     device=rt.device)
        return self.head.forward(h, logits_out)
