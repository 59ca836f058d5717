"""Mixer parts.  ``gqa``: causal grouped-query attention over the cache.

Formulas: q, k, v projections with optional biases (src/model/transformer.cpp:245-250;
src/model/model.cpp:145-152); query head hh reads kv head hh / (heads / kv_heads)
(src/model/transformer.cpp:264); scores scaled by 1/sqrt(head_dim) after the dot (:235, :271);
causal by position (:270); softmax and weighted sum (:273-280); output projection without
bias added to the residual stream (:283-284).  The three projections are stored as one
matrix [q; k; v] so that one product serves them.
"""
from __future__ import annotations

import math

import torch

from ..cache.storage import KVRequest
from ..ops import kernels
from .registry import TensorDecl, nested_build, nested_declare, part


@part("mixer", "gqa")
class GQAttention:
    """params: ``width``, ``n_heads``, ``n_kv_heads``, ``head_dim``, ``bias`` (q/k/v), ``window`` (0: all),
    ``scale`` (default 1/sqrt(head_dim)), ``position`` (a PartSpec of the position family)."""

    @classmethod
    def declare(cls, spec):
        p = spec.params
        q, kv, w = p["n_heads"] * p["head_dim"], p["n_kv_heads"] * p["head_dim"], p["width"]
        d = {"q_proj.weight": TensorDecl((q, w)), "k_proj.weight": TensorDecl((kv, w)),
             "v_proj.weight": TensorDecl((kv, w)), "o_proj.weight": TensorDecl((w, q))}
        if p.get("bias", False):
            d.update({"q_proj.bias": TensorDecl((q,), "bias"), "k_proj.bias": TensorDecl((kv,), "bias"),
                      "v_proj.bias": TensorDecl((kv,), "bias")})
        d.update(nested_declare("position", p["position"]))      # a position part may have tensors of its own
        return d

    def __init__(self, spec, tensors, rt, **_):
        p = spec.params
        self.rt = rt
        self.width = int(p["width"])
        self.n_heads, self.n_kv_heads, self.head_dim = int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        if self.n_heads % self.n_kv_heads:
            raise ValueError("gqa: n_heads must be a multiple of n_kv_heads")
        self.window = int(p.get("window", 0))
        self.scale = float(p.get("scale", 1.0 / math.sqrt(self.head_dim)))
        self.w_qkv = rt.to_compute(torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                                              tensors["v_proj.weight"]], dim=0))
        self.b_qkv = None
        if p.get("bias", False):
            self.b_qkv = rt.to_f32(torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]]))
        self.w_o = rt.to_compute(tensors["o_proj.weight"])
        self.position = nested_build("position", p["position"], tensors, rt)

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    defers_norm = True

    @property
    def takes_padding_rows(self) -> bool:
        """Token rows of no sequence (index -1) do no harm: the rotation skips them, attention gives them no job, and
        the products treat rows alone — if the position part agrees."""
        return bool(getattr(self.position, "takes_padding_rows", False))

    def step_plan(self, ctx, binding):
        """What of this step's launches depends on more than the step's padded shape (a recorded step is replayed
        only for a step with the same answer): the decode kernel's split and variant."""
        if not ctx.decode or self.rt.dtype != torch.bfloat16:
            return None
        g = binding.group
        S, P = ctx.pages_of(g).shape
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if g.page_size != 64 or not kernels.attention_decode_supported(hd, nh // nkv):
            return None
        return kernels.decode_plan_token(ctx, S, P, g.page_size, nkv, hd, nh // nkv)

    def forward(self, h, x, ctx, binding, then_norm=None) -> bool:
        T = h.shape[0]
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        qkv = self.rt.scratch("qkv", (T, (nh + 2 * nkv) * hd))
        kernels.linear(h, self.w_qkv, qkv, self.b_qkv)
        attn = self.rt.scratch("attn_out", (T, nh * hd))
        g = binding.group
        pages = ctx.pages_of(g)
        fused = self.position.fused_rotation()
        if fused is not None and kernels.attention_fuses_rotation(qkv, ctx, pages, g.page_size, nh, nkv, hd, fused[1], self.rt):
            rope = (fused[0], fused[1], binding.writes)        # a decode step: the attention kernel rotates and appends
        else:
            rope = None
            self.position.rotate_and_store(qkv, ctx, binding, nh, nkv, hd)
        kernels.attention(qkv, attn, g.k[binding.index], g.v[binding.index], ctx, pages, g.page_size,
                          nh, nkv, hd, self.scale, self.window, rt=self.rt, rope=rope)
        return kernels.linear(attn, self.w_o, x, None, kernels.OUT_ADD_F32, then_norm)
