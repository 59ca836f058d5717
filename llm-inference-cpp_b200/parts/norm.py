"""Norm parts.  ``rms``: y = weight · (x · rsqrt(mean(x²) + eps)), as src/model/kernels.cpp:115-120
computes it (scale first, then weight; plain weight, not 1 + weight), the sum of squares in fp32."""
from __future__ import annotations

from ..ops import kernels
from .registry import TensorDecl, part


@part("norm", "rms")
class RMSNorm:
    """params: ``width``, ``eps``.  tensors: ``weight [width]`` (kept in fp32)."""

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
