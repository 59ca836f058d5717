"""Arrangements of a layer.  ``prenorm``: x += mixer(norm(x)); x += ffn(norm(x))
(include/llmi/model/transformer.hpp:49-52).

Norm deferral (optional, see :class:`ops.kernels.DeferredNorm`): a mixer or feed-forward whose class sets
``defers_norm = True`` accepts a filled deferred norm as its input ``h`` and a keyword ``then_norm`` — a
deferred norm to fill with its last, residual-adding product — and returns whether it filled it.  The block
uses this where both neighbours of a norm take part and the norm offers ``deferred``; everything else runs
the norm the plain way, so parts without these extras work unchanged.
"""
from __future__ import annotations

from .registry import part


def _defers(p) -> bool:
    return bool(getattr(p, "defers_norm", False))


@part("block", "prenorm")
class PreNormBlock:
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone
    def __init__(self, mixer_norm, mixer, ffn_norm, ffn):
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    @property
    def entry_norm(self):
        """The norm this block applies to x first, if whoever updates x before the block may fill its
        deferred form (``forward(..., entry=)``); else None."""
        return self.mixer_norm if _defers(self.mixer) and hasattr(self.mixer_norm, "deferred") else None

    def forward(self, x, ctx, binding, entry=None, next_norm=None):
        """``entry``: the filled deferred form of this block's first norm, or None.  ``next_norm``: the norm
        that reads x after this block, or None.  Returns that norm's deferred form if the block filled it."""
        T = x.shape[0]
        h = entry if entry is not None else self.mixer_norm.forward(x)
        then = None
        if _defers(self.mixer) and _defers(self.ffn) and hasattr(self.ffn_norm, "deferred"):
            then = self.ffn_norm.deferred(T, "deferred_inner")
        if then is not None and self.mixer.forward(h, x, ctx, binding, then_norm=then):
            h = then
        else:
            if then is None:
                self.mixer.forward(h, x, ctx, binding)
            h = self.ffn_norm.forward(x)
        then = next_norm.deferred(T, "deferred_outer") if (next_norm is not None and _defers(self.ffn)) else None
        if then is not None:
            return then if self.ffn.forward(h, x, ctx, then_norm=then) else None
        self.ffn.forward(h, x, ctx)
        return None
