"""Position-encoding parts.

``rotary_half``: inv_freq[i] = 1 / theta^(2i/d) in fp32 (src/model/transformer.cpp:59-65);
pairs (i, i + d/2) rotated by angle = float(pos) · inv_freq[i] (src/model/kernels.cpp:122-134);
applied to q and k, never to v; k is stored rotated (src/model/transformer.cpp:251-262).
``none``: keys and values are stored as they are.

A position part that acts elsewhere (say, a table added to the embeddings) overrides
``at_embedding`` and keeps ``rotary_dim = 0``.
"""
from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from .registry import part


class PositionEncoding:
    rotary_dim = 0
    inv_freq = None

    @classmethod
    def declare(cls, spec):
        return {}

    def at_embedding(self, x, ctx) -> None:
        """Hook after the embedding lookup; the default adds nothing."""

    def fused_rotation(self):
        """(inv_freq, rotary_dim) if all this part does to q, k, v is the rotation of pairs and the append that
        :meth:`rotate_and_store` does — a mixer may then let its attention kernel do both; None for a
        subclass with a ``rotate_and_store`` of its own."""
        if type(self).rotate_and_store is not PositionEncoding.rotate_and_store:
            return None
        return self.inv_freq, self.rotary_dim

    def rotate_and_store(self, qkv, ctx, binding, n_heads, n_kv_heads, head_dim) -> None:
        """Rotate q (in place) and k by position and append k, v to the call's cache pages."""
        g = binding.group
        kernels.rope_store(qkv, self.inv_freq, self.rotary_dim, ctx.tok_seq, ctx.tok_pos, ctx.pages_of(g),
                           g.page_size, g.k[binding.index], g.v[binding.index], n_heads, n_kv_heads, head_dim,
                           write_kv=binding.writes)


@part("position", "none")
class NoPosition(PositionEncoding):
    takes_padding_rows = True       # (a step padded to a shape has token rows of no sequence: see engine/graphs.py)

    def __init__(self, spec, tensors, rt, **_):
        pass


@part("position", "rotary_half")
class RotaryHalf(PositionEncoding):
    """params: ``head_dim``, ``theta``, optional ``rotary_dim`` (default: the whole head)."""
    takes_padding_rows = True       # the rotation kernel skips rows of no sequence

    def __init__(self, spec, tensors, rt, **_):
        d = int(spec.params.get("rotary_dim", spec.params["head_dim"]))
        if d % 2 or d > int(spec.params["head_dim"]):
            raise ValueError("rotary_half: rotary_dim must be even and at most head_dim")
        theta = np.float32(spec.params["theta"])
        exponent = (np.arange(0, d, 2, dtype=np.float32)) / np.float32(d)
        inv = (np.float32(1.0) / np.power(theta, exponent, dtype=np.float32)).astype(np.float32)
        self.rotary_dim = d
        self.inv_freq = torch.from_numpy(inv).to(rt.device)
