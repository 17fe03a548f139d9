"""Architecture-neutral description of a model: which parts each layer is made
of, in which order layers run, and which checkpoint tensor feeds which part.

An architecture's typed configuration (see ``llama.py``) turns its own
``config.json`` keys into one :class:`ModelSpec`.  Everything below the spec
(parts, cache, step function) reads sizes and constants from here and never
asks which architecture it is serving.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: ``kind`` is a key of the matching part registry,
    ``params`` are the constructor arguments (sizes, constants), ``tensors``
    maps the part's own tensor keys to checkpoint tensor names."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    tensors: Dict[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A residual block: an arrangement ``block`` (a key of the block registry)
    and the parts it arranges, by the names that arrangement gives them.  The
    ``prenorm`` arrangement has ``mixer_norm``, ``mixer``, ``feed_forward_norm``
    and ``feed_forward``; another arrangement (four norms, two mixers side by
    side) names its own."""

    block: str
    parts: Dict[str, PartSpec]

    def part(self, name: str) -> PartSpec:
        if name not in self.parts:
            raise KeyError(f"block {self.block!r} needs a part named {name!r}; "
                           f"the layer has {sorted(self.parts)}")
        return self.parts[name]

    def with_parts(self, **parts: PartSpec) -> "LayerSpec":
        """A copy with some parts replaced or added."""
        return LayerSpec(self.block, {**self.parts, **parts})


@dataclass(frozen=True)
class RunEntry:
    """One execution of a layer inside a step.  ``layer`` indexes
    ``ModelSpec.layers``; the same layer may appear in several entries.
    ``reads_cache_of`` names an earlier entry (by its index in the run order)
    whose cache this entry reads instead of owning one."""

    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_positions: int
    embedding: PartSpec
    layers: List[LayerSpec]
    run_order: List[RunEntry]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run_order[{i}] names layer {e.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if e.reads_cache_of is not None:
                j = e.reads_cache_of
                if not 0 <= j < i:
                    raise ValueError(
                        f"run_order[{i}] reads the cache of entry {j}, which "
                        f"does not run before it")
                if self.run_order[j].reads_cache_of is not None:
                    raise ValueError(
                        f"run_order[{i}] reads the cache of entry {j}, which "
                        f"owns no cache itself")
