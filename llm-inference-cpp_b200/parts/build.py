"""From a ModelSpec and named tensors to live parts, and the table of tensors a spec expects.

The reference lists its expected tensors in one function for its one model
(src/model/model.cpp:135-162).  Here every part declares its own tensors under
its prefix, and the table of a model is the union over its parts, in the order
the parts appear.
"""
from __future__ import annotations

from . import attention, block, embedding, feedforward, norm, position  # noqa: F401  (register the built-in parts)
from .registry import TensorDecl, get_part
from .spec import ModelSpec, PartSpec


def _part_specs(spec: ModelSpec):
    yield "embedding", spec.embedding
    for layer in spec.layers:
        for _, family, ps in layer.slots():
            yield family, ps
    yield "norm", spec.final_norm
    yield "head", spec.head


def expected_tensors(spec: ModelSpec) -> dict:
    """Full tensor name -> TensorDecl for everything the model reads from its weight file."""
    out: dict[str, TensorDecl] = {}
    for family, ps in _part_specs(spec):
        for local, decl in get_part(family, ps.kind).declare(ps).items():
            name = ps.prefix + local
            if name in out and out[name].shape != decl.shape:
                raise ValueError(f"tensor {name} is declared twice with different shapes")
            out[name] = decl
    return out


def _make(family: str, ps: PartSpec, tensors: dict, rt, **context):
    cls = get_part(family, ps.kind)
    local = {name: tensors[ps.prefix + name] for name in cls.declare(ps)}
    return cls(ps, local, rt, **context)


class NoMixer:
    """Stands in for the mixer of a layer that has none: it keeps no cache."""
    takes_padding_rows = True       # token rows of no sequence (a step padded to a shape) do no harm: rows are treated alone

    def cache_request(self):
        return None


class BuiltLayer:
    def __init__(self, block_part, parts: dict):
        self.block = block_part
        self.parts = parts                              # slot -> built part
        self.mixer = parts.get("mixer") or NoMixer()    # the part whose cache the layer keeps


def build_parts(spec: ModelSpec, tensors: dict, rt):
    """-> (embedding, [BuiltLayer], final_norm, head)."""
    emb = _make("embedding", spec.embedding, tensors, rt)
    layers = []
    for i, ls in enumerate(spec.layers):
        parts = {slot: _make(family, ps, tensors, rt) for slot, family, ps in ls.slots()}
        try:
            block = get_part("block", ls.block)(**parts)
        except TypeError as e:
            raise ValueError(f"layer {i}: the arrangement {ls.block!r} does not take the slots {sorted(parts)}: {e}") from None
        layers.append(BuiltLayer(block, parts))
    final_norm = _make("norm", spec.final_norm, tensors, rt)
    head = _make("head", spec.head, tensors, rt, embedding=emb)
    return emb, layers, final_norm, head
