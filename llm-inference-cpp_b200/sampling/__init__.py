"""Choosing the next token: greedy, or temperature with top-k and top-p.

Options and their meaning are the reference's (include/llmi/model/sampling.hpp:11-24;
src/model/sampling.cpp:11-76): ``temperature <= 0`` is greedy (the first maximum);
otherwise softmax(logits / temperature), then ``top_k`` (0: off), then ``top_p`` (1: off),
renormalised, then an inverse-CDF draw in ascending id order.  The choice runs on the
device (``csrc/sampling.cu``); only the uniform numbers are made on the host.

The reference draws from one ``std::mt19937_64`` per process (apps/llmi-chat/main.cpp:109),
so a sequence's draws depend on what was generated before it.  Here every request has a
stream of its own, keyed by (seed, request index): a request's tokens do not depend on its
batch-mates.  As with the reference, a seed reproduces this engine only
(docs/sampling.md:21-27).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..ops import kernels


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0      # the command lines' default is greedy (apps/llmi-generate/main.cpp:222)
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


class UniformStream:
    """The uniform numbers in [0, 1) of one request, reproducible from (seed, request index)."""

    def __init__(self, seed: int, request_index: int):
        self._gen = np.random.Generator(np.random.Philox(key=[seed & (2**64 - 1), request_index & (2**64 - 1)]))

    def next(self) -> float:
        return float(self._gen.random())


class Sampler:
    """Device-side choice for the rows of a logits matrix."""

    def __init__(self, params: SamplingParams, rt):
        self.params = params
        self.rt = rt
        self._u_host = None

    def prepare(self, n_rows: int, streams=None) -> None:
        """Host side of a choice: draw one uniform number per real row and copy them to the device.
        (Kept apart from ``launch`` so that the launch can be recorded in a CUDA graph.)"""
        if self.params.greedy:
            return
        if streams is None or len(streams) > n_rows:
            raise ValueError("sampling needs one uniform stream per row")
        if self._u_host is None or self._u_host.numel() < n_rows:
            self._u_host = torch.empty(max(n_rows, 64), dtype=torch.float64, pin_memory=True)
        u_np = self._u_host.numpy()
        u_np[:n_rows] = 0.5
        for i, s in enumerate(streams):
            u_np[i] = s.next()
        u_dev = self.rt.scratch("sample_uniforms", (max(n_rows, 64),), torch.float64)
        u_dev[:n_rows].copy_(self._u_host[:n_rows], non_blocking=True)

    def launch(self, logits: torch.Tensor, n_rows: int | None = None) -> torch.Tensor:
        """Device side of a choice: logits fp32 [R, V] -> int32 [R] (scratch, valid until the next call)."""
        R, V = logits.shape
        out = self.rt.scratch("sampled_ids", (max(R, 64),), torch.int32)[:R]
        p = self.params
        if p.greedy:
            kernels.argmax(logits, out)
            return out
        u_dev = self.rt.scratch("sample_uniforms", (max(R, 64),), torch.float64)
        probs = self.rt.scratch("sample_probs", (R, V), torch.float32)
        kernels.sample(logits, float(p.temperature), int(p.top_k), float(p.top_p), u_dev, probs, out)
        return out

    def choose(self, logits: torch.Tensor, streams=None) -> torch.Tensor:
        """logits fp32 [R, V] -> int32 [R] on the device; ``streams``: one UniformStream per row."""
        self.prepare(logits.shape[0], streams)
        return self.launch(logits)
