"""Registries of part kinds, one per family, and the interface each family keeps.

Families and what the engine calls on their members (``rt`` is the
:class:`~..engine.runtime.Runtime`, ``ctx`` the step's
:class:`~..engine.batch.StepContext`, ``x`` the fp32 residual stream
``[tokens, width]``, ``h`` a normalised copy of it in the compute type):

``norm``       ``forward(x, rows=None) -> h``
``position``   held by another part through its params (``"position": PartSpec``), with tensors of its
               own if it declares any: by a mixer that keeps keys and values, which calls
               ``rotate_and_store(qkv, ctx, binding, n_heads, n_kv_heads, head_dim)``, or by the
               embedding, which calls ``at_embedding(x, ctx)`` after the lookup (may add to ``x``)
``mixer``      ``cache_request() -> KVRequest | StateRequest | None`` and
               ``forward(h, x, ctx, binding)``: adds its output to ``x``
``ffn``        ``forward(h, x, ctx)``: adds its output to ``x``
``block``      ``forward(x, ctx, binding)``: one layer's arrangement of the above; built with one keyword argument
               per filled slot of its ``LayerSpec`` (``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn`` and whatever
               the spec adds under ``more``)
``embedding``  ``forward(token_ids, ctx) -> x`` and ``table()`` (for a tied head)
``head``       ``forward(h_rows) -> logits fp32 [rows, vocab]``

Every member also has ``declare(spec) -> {local tensor name: TensorDecl}`` (a
classmethod: what it reads from the weight file under ``spec.prefix``) and is
constructed as ``cls(spec, tensors, rt, **context)`` with its declared tensors.
No part knows which model it is in.

Optional extras, for fusions that cross two parts.  A part without them works unchanged; the caller falls
back to the plain path.

``position``   ``fused_rotation() -> (inv_freq, rotary_dim) | None``: all the part does to q, k, v is the
               rotation of pairs and the append of ``rotate_and_store``, so a mixer may let its attention
               kernel do both.
``norm``       ``deferred(n_tokens, name) -> kernels.DeferredNorm | None``: the norm split over the products
               around it (the one before fills it, the one after applies the scale).
``mixer``/``ffn``  class attribute ``defers_norm = True``: ``forward`` accepts a filled ``DeferredNorm`` as
               ``h`` and a keyword ``then_norm=`` (a ``DeferredNorm`` to fill with the part's last,
               residual-adding product) and returns whether it filled it.
``block``      property ``entry_norm`` (the norm it applies first, if the block before may fill its deferred
               form) and ``forward(x, ctx, binding, entry=None, next_norm=None) -> DeferredNorm | None``.
``mixer``      ``step_plan(ctx, binding) -> hashable | None``: what the part's launches for this step depend on
               beside the step's padded shape (its attention kernel's split, which follows the live sequences).
               A recorded decode step is replayed only for a step whose mixers give the same answers.
any part       class attribute ``takes_padding_rows = True``: token rows that belong to no sequence (index -1)
               do it no harm, so its model's short prompt steps may be padded to a shape and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass

FAMILIES = ("norm", "position", "mixer", "ffn", "block", "embedding", "head")
_PARTS: dict[str, dict[str, type]] = {f: {} for f in FAMILIES}


@dataclass(frozen=True)
class TensorDecl:
    shape: tuple
    # "matrix" | "norm_scale" | "bias" | "table": floating tensors (the role says how random weights draw them);
    # "int_table": the only role a file may store as integers
    role: str = "matrix"


def register_part(family: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if family not in _PARTS:
        raise ValueError(f"unknown part family {family!r}; families are {FAMILIES}")
    if kind in _PARTS[family] and not replace:
        raise ValueError(f"{family} part {kind!r} is already registered")
    _PARTS[family][kind] = cls


def get_part(family: str, kind: str) -> type:
    try:
        return _PARTS[family][kind]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(family, {}))) or "none"
        raise KeyError(f"no {family} part of kind {kind!r} is registered (known: {known})") from None


def nested_declare(family: str, ps) -> dict:
    """The tensors of a part that another part holds in its params (a mixer's or an embedding's position
    part): its own declarations under its own prefix, which is relative to the holder's."""
    return {ps.prefix + name: decl for name, decl in get_part(family, ps.kind).declare(ps).items()}


def nested_build(family: str, ps, tensors: dict, rt, **context):
    """Build such a part from the holder's tensors (see :func:`nested_declare`)."""
    cls = get_part(family, ps.kind)
    return cls(ps, {name: tensors[ps.prefix + name] for name in cls.declare(ps)}, rt, **context)


def part(family: str, kind: str):
    """Class decorator: ``@part("mixer", "gqa")``."""
    def deco(cls):
        register_part(family, kind, cls)
        cls.family, cls.kind = family, kind
        return cls
    return deco
