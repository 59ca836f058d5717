"""Seeded random weights for any registered architecture, and a writer of model folders.

The reference builds random models only in its tests
(tests/transformer_test.cpp:162-197: normal matrices, norm weights around one,
written as an in-memory safetensors blob).  Here it is a mode of the library:
matrices, tables and biases are N(0, 0.02), norm scales are 1 + N(0, 0.1), each
tensor drawn from its own generator keyed by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are made.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from ..config.registry import parse_config
from ..parts.build import expected_tensors
from .safetensors_io import write_safetensors

MATRIX_STD = 0.02
NORM_STD = 0.1


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, shape, role: str, seed: int, device="cpu") -> torch.Tensor:
    """One fp32 tensor of the given role, reproducible from (seed, name) on a given device type."""
    if role not in ("matrix", "norm_scale", "bias", "table"):
        raise ValueError(f"random weights: no rule for a tensor of role {role!r} ({name})")
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    noise = torch.randn(tuple(shape), generator=gen, device=device, dtype=torch.float32)
    if role == "norm_scale":
        return 1.0 + NORM_STD * noise
    return MATRIX_STD * noise


def random_tensors(spec, seed: int, device="cpu", dtype=torch.float32) -> dict:
    """All tensors a ModelSpec expects, drawn in fp32 and rounded once to ``dtype``."""
    return {name: random_tensor(name, d.shape, d.role, seed, device).to(dtype)
            for name, d in expected_tensors(spec).items()}


def write_random_model(model_dir: str, config: dict, seed: int, dtype=torch.float32) -> str:
    """Write ``config.json`` and ``model.safetensors`` for a config.json dict and a seed."""
    arch, cfg = parse_config(config)
    spec = arch.model_spec(cfg)
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(config), f, indent=1)
    tensors = random_tensors(spec, seed, "cpu", dtype)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return model_dir
