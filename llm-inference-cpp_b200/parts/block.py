"""Arrangements of a layer.  ``prenorm``: x += mixer(norm(x)); x += ffn(norm(x))
(include/llmi/model/transformer.hpp:49-52)."""
from __future__ import annotations

from .registry import part


@part("block", "prenorm")
class PreNormBlock:
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def forward(self, x, ctx, binding) -> None:
        h = self.mixer_norm.forward(x)
        self.mixer.forward(h, x, ctx, binding)
        h = self.ffn_norm.forward(x)
        self.ffn.forward(h, x, ctx)
