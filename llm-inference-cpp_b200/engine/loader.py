"""From a model folder, or from a configuration and a seed, to a :class:`Model` on the device.

A folder holds ``config.json`` and one ``model.safetensors`` (src/model/model.cpp:216-224).
The architecture named in config.json picks the recipe from the registry; the file is
checked against the tensors that recipe's parts declare before anything is copied.
"""
from __future__ import annotations

import os

import torch

from .. import models  # noqa: F401  (registers the architectures)
from ..config.registry import parse_config, read_model_config
from ..parts.build import expected_tensors
from ..weights.binding import load_tensors
from ..weights.random_weights import random_tensors
from ..weights.safetensors_io import SafetensorsFile
from .model import Model

_DTYPES = {"float32": torch.float32, "fp32": torch.float32, "f32": torch.float32,
           "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {name!r}") from None


def load_model(model_dir: str, dtype="bfloat16", device="cuda:0") -> Model:
    arch, cfg = read_model_config(model_dir)
    spec = arch.model_spec(cfg)
    decls = expected_tensors(spec)
    f = SafetensorsFile(os.path.join(model_dir, "model.safetensors"))
    try:
        tensors = load_tensors(f, decls, device, arch.tolerated_extra_tensors)
    finally:
        f.close()
    return Model(spec, tensors, parse_dtype(dtype), device, config=cfg)


def random_model(config: dict, seed: int = 0, dtype="bfloat16", device="cuda:0", on_device: bool = False) -> Model:
    """A model with seeded random weights, without a folder.

    The weights are drawn in fp32 and rounded once to the compute type.  With
    ``on_device`` they are drawn by the device's generator (fast for large models, but a
    different stream of numbers than the folder writer's CPU generator).
    """
    arch, cfg = parse_config(config)
    spec = arch.model_spec(cfg)
    dt = parse_dtype(dtype)
    tensors = random_tensors(spec, seed, device if on_device else "cpu", dt)
    return Model(spec, tensors, dt, device, config=cfg)
