"""Descriptions of a model as data: which part runs where, with which sizes.

An architecture turns its typed configuration into a :class:`ModelSpec`.  The
builder (``parts.build``) turns a ModelSpec plus named tensors into live parts.
Nothing below names a model: a part is a *kind* (a key of the part registries),
its *params* (sizes and constants) and the *prefix* of its tensor names.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


@dataclass(frozen=True)
class PartSpec:
    kind: str                       # key in the registry of its family
    params: dict = field(default_factory=dict)
    prefix: str = ""                # tensor names of the part start with this


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) and the parts it arranges, each in a named slot.

    The four usual slots have fields of their own; any of them may be None (a layer without a
    feed-forward, say), and ``more`` adds slots by name — ``(slot, family, PartSpec)`` triples, for an
    arrangement with further norms or a second feed-forward.  The block class is built with one keyword
    argument per filled slot.  The part in the slot ``mixer``, if any, is the one whose cache the layer keeps.
    """
    block: str                      # arrangement, e.g. "prenorm"
    mixer_norm: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    more: tuple = ()                # ((slot, family, PartSpec), ...)

    def slots(self):
        """(slot, family, PartSpec) of every filled slot, in the order the tensors are declared."""
        for slot, family in (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("ffn", "ffn")):
            ps = getattr(self, slot)
            if ps is not None:
                yield slot, family, ps
        for slot, family, ps in self.more:
            if slot in ("mixer_norm", "mixer", "ffn_norm", "ffn", "block", "more"):
                raise ValueError(f"layer: the slot name {slot!r} is taken")
            yield slot, family, ps


@dataclass(frozen=True)
class ScheduleEntry:
    """One call in the order layers run.

    ``layer`` indexes ``ModelSpec.layers``; the same layer may be named twice.
    ``cache_of`` names the schedule position whose cache this call reads instead
    of keeping one of its own (None: its own).  A call that reads another call's
    cache writes nothing into it.
    """
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: PartSpec
    layers: tuple
    schedule: tuple
    final_norm: PartSpec
    head: PartSpec
    stop_ids: tuple = ()
    extra: Any = None
