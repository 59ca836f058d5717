"""Norm parts.  ``rms``: y = weight · (x · rsqrt(mean(x²) + eps)), as src/model/kernels.cpp:115-120
computes it (scale first, then weight; plain weight, not 1 + weight), the sum of squares in fp32."""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("norm", "rms")
class RMSNorm:
    """params: ``width``, ``eps``.  tensors: ``weight [width]`` (kept in fp32)."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    @classmethod
    def declare(cls, spec):
        return {"weight": TensorDecl((spec.params["width"],), "norm_scale")}

    def __init__(self, spec, tensors, rt, **_):
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = rt.to_f32(tensors["weight"])
        self.rt = rt

    def forward(self, x, rows=None, scratch_name: str = "norm_out"):
        """x fp32 [tokens, width] -> normalised rows in the compute type; ``rows`` picks input rows."""
        n = x.shape[0] if rows is None else rows.shape[0]
        out = self.rt.scratch(scratch_name, (n, self.width))
        kernels.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

    def deferred(self, n_tokens: int, name: str):
        """This norm for ``n_tokens`` rows as a :class:`kernels.DeferredNorm` — to be filled by the product
        that updates x and read by the product after the norm — or None when the step's size or type does
        not allow it (then :meth:`forward` is the way).  ``name`` keeps apart the buffers of norms that are
        in flight at the same time."""
        if not kernels.norm_deferrable(n_tokens, self.width, self.rt.dtype):
            return None
        h = self.rt.scratch(name + "_h", (n_tokens, self.width))
        ss = self.rt.scratch(name + "_ss", ((self.width + 15) // 16, kernels.DeferredNorm.SS_STRIDE), torch.float32)
        return kernels.DeferredNorm(self.weight, self.eps, h, ss)
