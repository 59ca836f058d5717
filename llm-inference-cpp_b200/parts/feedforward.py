"""Feed-forward parts.  ``swiglu``: x += (silu(h·Wgᵀ) ⊙ (h·Wuᵀ))·Wdᵀ, no biases
(src/model/transformer.cpp:288-292; silu(z) = z / (1 + exp(-z)), src/model/kernels.cpp:148).
Gate and up are stored as one matrix [gate; up] so that one product serves both."""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, part


@part("ffn", "swiglu")
class SwiGLU:
    """params: ``width``, ``inner``."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    @classmethod
    def declare(cls, spec):
        w, f = spec.params["width"], spec.params["inner"]
        return {"gate_proj.weight": TensorDecl((f, w)), "up_proj.weight": TensorDecl((f, w)),
                "down_proj.weight": TensorDecl((w, f))}

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self.width, self.inner = int(spec.params["width"]), int(spec.params["inner"])
        gate, up = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        # The tensor-core product can finish silu(gate)·up itself when gate and up rows alternate;
        # otherwise the rows are [gate; up] and a gating kernel follows the product.
        self.fused_gate = rt.dtype == torch.bfloat16 and self.width % 8 == 0 and not kernels._FORCE_SIMT
        if self.fused_gate:
            self.w_gate_up = rt.to_compute(torch.stack([gate, up], dim=1).reshape(2 * self.inner, self.width))
        else:
            self.w_gate_up = rt.to_compute(torch.cat([gate, up], dim=0))
        self.w_down = rt.to_compute(tensors["down_proj.weight"])

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_gate_up, self.w_down))

    defers_norm = True

    def forward(self, h, x, ctx, then_norm=None) -> bool:
        T = h.shape[0]
        act = self.rt.scratch("ffn_act", (T, self.inner))
        if self.fused_gate and kernels.gemm_tc_eligible(getattr(h, "h", h), self.w_gate_up):
            kernels.gemm_bf16(h, self.w_gate_up, act, None, kernels.OUT_SWIGLU)
        else:
            if self.fused_gate:
                raise kernels.KernelError("swiglu: activations are not aligned for the tensor-core product")
            gate_up = self.rt.scratch("ffn_gate_up", (T, 2 * self.inner))
            kernels.linear(h, self.w_gate_up, gate_up)
            kernels.swiglu(gate_up, act)
        return kernels.linear(act, self.w_down, x, None, kernels.OUT_ADD_F32, then_norm)
