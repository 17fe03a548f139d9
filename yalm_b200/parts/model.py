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
    def cache_needs(self) -> Dict[int, CacheNeed]:
        """Run-entry index -> what its mixer asks of the cache (entries that
        read another entry's cache own none)."""
        needs = {}
        for i, e in enumerate(self.run_order):
            if e.reads_cache_of is not None:
                continue
            need = self.layers[e.layer].mixer.cache_need()
            if need is not None:
                needs[i] = need
        return needs

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
        for i, e in enumerate(self.run_order):
            layer = self.layers[e.layer]
            owner = i if e.reads_cache_of is None else e.reads_cache_of
            if owner not in views:
                need = self.layers[self.run_order[owner].layer].mixer.cache_need()
                view = cache.view(owner) if need is not None else None
                if view is not None and view.kind == "kv" and owner in self._readers:
                    view = dataclasses.replace(view, kv_step=rt.buffer(
                        f"kv_step_{owner}", (batch.n_tokens, 2, need.kv_heads, need.head_dim),
                        rt.dtype))
                views[owner] = view
            layer.forward(stream, batch, views[owner], shared=e.reads_cache_of is not None)
        if n_want == 0:
            return None
        h = self.final_norm(stream, rows=want_rows, n_rows=n_want, name="final_normed")
        if logits_out is None:
            logits_out = torch.empty((n_want, self.spec.vocab_size), dtype=torch.float32,
                                     device=rt.device)
        return self.head.forward(h, logits_out)
