"""Binding the tensors of a file to the tensors a model expects, by name.

The reference checks each expected tensor in turn and stops at the first fault
(src/model/model.cpp:177-202: ``missing tensor``, ``has shape``, ``has dtype``,
``unexpected tensor``).  Here all faults of a file are collected and reported in
one error, so that a wrong export shows everything that is wrong with it at once.

Storage rules on the device: floating matrices and vectors stored in 16 bits are
kept as bfloat16, a tensor stored in 32 bits stays 32-bit, integer tables become
int32.  What a part needs in another type (a matrix in the compute type, a norm
weight in fp32) it converts itself when it is built.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch

from .safetensors_io import SafetensorsFile

FLOAT_STORAGE = ("F32", "F16", "BF16")
INT_STORAGE = ("I32", "I64")


class WeightBindingError(ValueError):
    """Raised once per file, listing every missing, unexpected and ill-shaped tensor."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, where: str = "model"):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, found, expected)
        self.wrong_dtype = list(wrong_dtype)      # (name, found)
        lines = [f"{where}: weights do not match the configuration"]
        for n in self.missing:
            lines.append(f"  missing tensor {n}")
        for n, found, exp in self.wrong_shape:
            lines.append(f"  {n} has shape {list(found)}, expected {list(exp)}")
        for n, found in self.wrong_dtype:
            lines.append(f"  {n} has dtype {found}, expected F32, F16 or BF16")
        for n in self.unexpected:
            lines.append(f"  unexpected tensor {n}")
        super().__init__("\n".join(lines))


def check_tensors(expected: Mapping[str, tuple], found: Mapping[str, tuple],
                  tolerated: Callable[[str], bool] = lambda n: False, where: str = "model") -> None:
    """``expected``: name → shape.  ``found``: name → (storage dtype name, shape)."""
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, shape in expected.items():
        if name not in found:
            missing.append(name)
            continue
        dt, fshape = found[name]
        if tuple(fshape) != tuple(shape):
            wrong_shape.append((name, fshape, shape))
        if dt not in FLOAT_STORAGE and dt not in INT_STORAGE:
            wrong_dtype.append((name, dt))
    unexpected = [n for n in found if n not in expected and not tolerated(n)]
    if missing or wrong_shape or wrong_dtype or unexpected:
        raise WeightBindingError(missing, unexpected, wrong_shape, wrong_dtype, where)


def storage_form(t: torch.Tensor) -> torch.Tensor:
    """The type a stored tensor keeps on the device (see module docstring)."""
    if t.dtype in (torch.float16,):
        return t.to(torch.bfloat16)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8):
        return t.to(torch.int32)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    return t


def load_tensors(file: SafetensorsFile, expected: Mapping[str, tuple], device,
                 tolerated: Callable[[str], bool] = lambda n: False) -> dict:
    """Check the file against ``expected`` and copy the expected tensors to ``device``."""
    found = {n: (t.dtype, t.shape) for n, t in file.tensors.items()}
    check_tensors(expected, found, tolerated, where=file.path)
    out = {}
    for name in expected:
        host = storage_form(file.tensor(name))
        out[name] = host.to(device, non_blocking=False).contiguous()
    return out
