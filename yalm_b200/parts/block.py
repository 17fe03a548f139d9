"""Arrangements of a layer's parts.  ``prenorm``: x += mixer(norm(x)); then
x += ffn(norm(x)) -- the reference's block order (infer.cpp:257-386).

A block arrangement is a class with ``__init__(layer_spec, rt)`` (it builds the
parts it names from ``layer_spec.parts``), ``parts()`` (the built parts with
their specs, for weight binding), ``mixers()`` (the parts that may ask for cache,
by name) and ``forward(stream, batch, views, shared)``.  ``views`` maps a mixer's
name to what that mixer sees of the cache: one :class:`CacheView`, a dict of them
by need name when the mixer declared several needs, or None.
"""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, make_part, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec, rt):
        self.spec = layer_spec
        self.mixer_norm = make_part(NORMS, layer_spec.part("mixer_norm"), rt)
        self.mixer = make_part(MIXERS, layer_spec.part("mixer"), rt)
        self.ffn_norm = make_part(NORMS, layer_spec.part("feed_forward_norm"), rt)
        self.ffn = make_part(FEED_FORWARDS, layer_spec.part("feed_forward"), rt)

    def parts(self):
        """(part, its PartSpec) pairs, for weight binding."""
        s = self.spec
        return [(self.mixer_norm, s.part("mixer_norm")), (self.mixer, s.part("mixer")),
                (self.ffn_norm, s.part("feed_forward_norm")), (self.ffn, s.part("feed_forward"))]

    def mixers(self):
        """name -> mixer, for the cache's needs."""
        return {"mixer": self.mixer}

    def forward(self, stream, batch, views, shared: bool = False):
        """Returns what the mixer returned: None, or a cache write that the model makes
        once every run entry that reads this entry's cache has run."""
        h = self.mixer_norm(stream)
        later = self.mixer.forward(h, batch, stream, views["mixer"], shared=shared)
        h = self.ffn_norm(stream)
        self.ffn.forward(h, batch, stream)
        return later
