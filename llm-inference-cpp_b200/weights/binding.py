"""Binding the tensors of a file to the tensors a model expects, by name.

The reference checks each expected tensor in turn and stops at the first fault
(src/model/model.cpp:177-202: ``missing tensor``, ``has shape``, ``has dtype``,
``unexpected tensor``).  Here all faults of a file are collected and reported in
one error, so that a wrong export shows everything that is wrong with it at once.

Storage rules on the device: a tensor stored as BF16 is kept as bfloat16, one stored
in 32 bits stays 32-bit, and one stored as F16 stays float16 until the part that owns
it converts it — widening F16 to fp32 is exact, as in the reference
(src/model/safetensors.cpp:290-299), so the 32-bit path sees the file's very values and
the bf16 path rounds them once.  Integer tables become int32; they are accepted only
for a tensor whose role is ``int_table`` — everything a model multiplies with must be
F32, F16 or BF16 (src/model/model.cpp:185-187).  What a part needs in another type (a
matrix in the compute type, a norm weight in fp32) it converts itself when it is built.
"""
from __future__ import annotations

from typing import Callable, Mapping

import torch

from .safetensors_io import SafetensorsFile

FLOAT_STORAGE = ("F32", "F16", "BF16")
INT_STORAGE = ("I32", "I64")


class WeightBindingError(ValueError):
    """Raised once per file, listing every missing, unexpected and ill-shaped tensor."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, where: str = "model", integer_roles=()):
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
            want = "I32 or I64" if n in integer_roles else "F32, F16 or BF16"
            lines.append(f"  {n} has dtype {found}, expected {want}")
        for n in self.unexpected:
            lines.append(f"  unexpected tensor {n}")
        super().__init__("\n".join(lines))


def _shape_and_role(decl) -> tuple:
    """An expected tensor is given as a shape or as a declaration with ``shape`` and ``role``."""
    if hasattr(decl, "shape") and hasattr(decl, "role"):
        return tuple(decl.shape), decl.role
    return tuple(decl), "matrix"


def check_tensors(expected: Mapping[str, tuple], found: Mapping[str, tuple],
                  tolerated: Callable[[str], bool] = lambda n: False, where: str = "model") -> None:
    """``expected``: name → shape, or → a declaration with ``shape`` and ``role``.
    ``found``: name → (storage dtype name, shape)."""
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, decl in expected.items():
        if name not in found:
            missing.append(name)
            continue
        shape, role = _shape_and_role(decl)
        dt, fshape = found[name]
        if tuple(fshape) != shape:
            wrong_shape.append((name, fshape, shape))
        if dt not in (INT_STORAGE if role == "int_table" else FLOAT_STORAGE):
            wrong_dtype.append((name, dt))
    unexpected = [n for n in found if n not in expected and not tolerated(n)]
    if missing or wrong_shape or wrong_dtype or unexpected:
        integer = {n for n, d in expected.items() if _shape_and_role(d)[1] == "int_table"}
        raise WeightBindingError(missing, unexpected, wrong_shape, wrong_dtype, where, integer)


def storage_form(t: torch.Tensor) -> torch.Tensor:
    """The type a stored tensor keeps on the device (see module docstring)."""
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
