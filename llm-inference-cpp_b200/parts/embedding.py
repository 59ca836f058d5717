"""Embedding and output-head parts.

``token_table``: x[t] = E[token[t]], no scaling (src/model/transformer.cpp:214-217).
``linear_head``: logits = h · Wᵀ with W the head matrix, or the embedding table when tied
(src/model/transformer.cpp:301-305); logits are fp32.
"""
from __future__ import annotations

import torch

from ..ops import kernels
from .registry import TensorDecl, nested_build, nested_declare, part


@part("embedding", "token_table")
class TokenTable:
    """params: ``vocab``, ``width``, optional ``position`` (a PartSpec of the position family whose
    ``at_embedding`` acts on the looked-up rows).  tensors: ``weight [vocab, width]`` and the position part's."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    @classmethod
    def declare(cls, spec):
        d = {"weight": TensorDecl((spec.params["vocab"], spec.params["width"]), "table")}
        if spec.params.get("position") is not None:
            d.update(nested_declare("position", spec.params["position"]))
        return d

    def __init__(self, spec, tensors, rt, **_):
        self.rt = rt
        self.vocab, self.width = int(spec.params["vocab"]), int(spec.params["width"])
        self.weight = rt.to_compute(tensors["weight"])
        pos = spec.params.get("position")
        self.position = nested_build("position", pos, tensors, rt) if pos is not None else None

    def table(self):
        return self.weight

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, token_ids, ctx):
        x = self.rt.scratch("residual", (token_ids.shape[0], self.width), torch.float32)
        kernels.embed(self.weight, token_ids, x)
        if self.position is not None:
            self.position.at_embedding(x, ctx)
        return x


@part("head", "linear_head")
class LinearHead:
    """params: ``vocab``, ``width``, ``tied``.  tensors: ``weight [vocab, width]`` unless tied."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    @classmethod
    def declare(cls, spec):
        if spec.params.get("tied", False):
            return {}
        return {"weight": TensorDecl((spec.params["vocab"], spec.params["width"]))}

    def __init__(self, spec, tensors, rt, embedding=None, **_):
        self.rt = rt
        self.vocab, self.width = int(spec.params["vocab"]), int(spec.params["width"])
        self.tied = bool(spec.params.get("tied", False))
        if self.tied:
            if embedding is None:
                raise ValueError("linear_head: a tied head needs the embedding part")
            self.weight = embedding.table()
        else:
            self.weight = rt.to_compute(tensors["weight"])

    def weight_bytes(self) -> int:
        return 0 if self.tied else self.weight.numel() * self.weight.element_size()

    def forward(self, h_rows):
        logits = self.rt.scratch("logits", (h_rows.shape[0], self.vocab), torch.float32)
        kernels.linear(h_rows, self.weight, logits, None, kernels.OUT_STORE_F32)
        return logits
