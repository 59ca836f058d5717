"""What every part shares at run time: the compute type, the device and named scratch buffers.

The reference allocates its temporaries anew in every call
(src/model/transformer.cpp:223-233) and notes the cost (docs/performance.md:128-130).
Here a scratch buffer is kept under a name and only grows; a step that needs no
more than an earlier one allocates nothing.  ``generation`` counts reallocations, so
that recorded CUDA graphs, which hold raw addresses, know when they are stale.
"""
from __future__ import annotations

import torch


class Runtime:
    def __init__(self, dtype: torch.dtype, device):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute type must be float32 or bfloat16, not {dtype}")
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("this library runs on a CUDA device only; there is no CPU path")
        self._buffers: dict[str, torch.Tensor] = {}
        self.generation = 0

    def scratch(self, name: str, shape, dtype=None) -> torch.Tensor:
        dtype = dtype or self.dtype
        n = 1
        for s in shape:
            n *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            grow = n if buf is None or buf.dtype != dtype else max(n, 2 * buf.numel())
            buf = torch.empty(grow, dtype=dtype, device=self.device)
            self._buffers[name] = buf
            self.generation += 1
        return buf[:n].view(*shape)

    def to_compute(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix in the compute type (bf16 stays bf16; widening to fp32 is exact)."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def to_f32(self, t: torch.Tensor) -> torch.Tensor:
        return t.to(device=self.device, dtype=torch.float32).contiguous()
