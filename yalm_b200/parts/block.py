"""Arrangements of a layer's parts.  ``prenorm``: x += mixer(norm(x)); then
x += ffn(norm(x)) -- the reference's block order (infer.cpp:257-386)."""
from __future__ import annotations

from .base import FEED_FORWARDS, MIXERS, NORMS, make_part, register_block


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, layer_spec, rt):
        self.mixer_norm = make_part(NORMS, layer_spec.mixer_norm, rt)
        self.mixer = make_part(MIXERS, layer_spec.mixer, rt)
        self.ffn_norm = make_part(NORMS, layer_spec.feed_forward_norm, rt)
        self.ffn = make_part(FEED_FORWARDS, layer_spec.feed_forward, rt)
        self.spec = layer_spec

    def parts(self):
        """(part, its PartSpec) pairs, for weight binding."""
        s = self.spec
        return [(self.mixer_norm, s.mixer_norm), (self.mixer, s.mixer),
                (self.ffn_norm, s.feed_forward_norm), (self.ffn, s.feed_forward)]

    def forward(self, stream, batch, view, shared: bool = False) -> None:
        h = self.mixer_norm(stream)
        self.mixer.forward(h, batch, stream, view, shared=shared)
        h = self.ffn_norm(stream)
        self.ffn.forward(h, batch, stream)
