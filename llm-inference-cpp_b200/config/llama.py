"""Typed configuration of the Llama / SmolLM2 dense decoder.

Every number the model needs comes from the architecture's own ``config.json``
keys; nothing is hard-wired.  The accepted keys, their defaults and the
rejections follow the reference parser (src/model/model.cpp:60-133):

* ``architectures`` must list exactly one name (model.cpp:66-77).
* ``vocab_size``, ``hidden_size``, ``intermediate_size``, ``num_hidden_layers``,
  ``num_attention_heads``, ``max_position_embeddings`` are required positive
  integers with upper bounds (model.cpp:25-28, 84-90).
* ``num_key_value_heads`` defaults to ``num_attention_heads`` (model.cpp:89).
* ``rms_norm_eps`` and ``rope_theta`` are required and positive (model.cpp:91-92).
* ``tie_word_embeddings`` and ``attention_bias`` default to false (model.cpp:93-95).
* ``hidden_act`` must be ``"silu"`` when present (model.cpp:110-112).
* ``eos_token_id`` may be a number, a list, null or absent (model.cpp:113-125).
* ``rope_scaling`` non-null and ``use_sliding_window`` true are errors
  (model.cpp:126-131).

One deliberate widening: ``head_dim`` is an independent size here.  The
reference insists on ``hidden_size / num_attention_heads`` (model.cpp:101-107);
this library only uses that quotient as the default when the key is absent,
because every projection shape is already written as ``heads * head_dim``
(model.cpp:137-138).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from typing import Any, Mapping

MAX_DIM = 1 << 20
MAX_VOCAB = 1 << 22
MAX_LAYERS = 1024
MAX_POSITIONS = 1 << 24
MAX_CONFIG_BYTES = 1 << 20


class ConfigError(ValueError):
    """A config.json that this library cannot run; the text says which key."""


def _get_uint(root: Mapping[str, Any], key: str, limit: int, fallback: int | None = None) -> int:
    v = root.get(key)
    if v is None:
        if fallback is not None:
            return fallback
        raise ConfigError(f'config: missing "{key}"')
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0 or v > limit:
        raise ConfigError(f'config: "{key}" must be an integer in 1..{limit}')
    return v


def _get_positive(root: Mapping[str, Any], key: str) -> float:
    if key not in root:
        raise ConfigError(f'config: missing "{key}"')
    v = root[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not v > 0:
        raise ConfigError(f'config: "{key}" must be a positive number')
    return float(v)


def _get_bool(root: Mapping[str, Any], key: str, fallback: bool) -> bool:
    v = root.get(key)
    if v is None:
        return fallback
    if not isinstance(v, bool):
        raise ConfigError(f'config: "{key}" must be true or false')
    return v


def _reject_duplicate_keys(pairs):
    seen = {}
    for k, v in pairs:
        if k in seen:
            raise ConfigError(f'config: duplicate key "{k}"')
        seen[k] = v
    return seen


def read_config_json(text: str) -> dict:
    """Parse config.json text into a dict; duplicate keys and non-objects are errors."""
    try:
        root = json.loads(text, object_pairs_hook=_reject_duplicate_keys)
    except json.JSONDecodeError as e:
        raise ConfigError(f"config: {e}") from None
    if not isinstance(root, dict):
        raise ConfigError("config: not a JSON object")
    return root


def architecture_name(root: Mapping[str, Any]) -> str:
    archs = root.get("architectures")
    if not isinstance(archs, list) or len(archs) != 1 or not isinstance(archs[0], str):
        raise ConfigError('config: "architectures" must list exactly one architecture')
    return archs[0]


@dataclass(frozen=True)
class LlamaConfig:
    """Sizes and constants of one Llama-architecture model (model.hpp:21-36)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    eos_token_ids: tuple[int, ...] = field(default_factory=tuple)
    architecture: str = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, root: Mapping[str, Any]) -> "LlamaConfig":
        arch = architecture_name(root)
        vocab = _get_uint(root, "vocab_size", MAX_VOCAB)
        hidden = _get_uint(root, "hidden_size", MAX_DIM)
        inter = _get_uint(root, "intermediate_size", MAX_DIM)
        layers = _get_uint(root, "num_hidden_layers", MAX_LAYERS)
        heads = _get_uint(root, "num_attention_heads", MAX_DIM)
        kv_heads = _get_uint(root, "num_key_value_heads", MAX_DIM, heads)
        max_pos = _get_uint(root, "max_position_embeddings", MAX_POSITIONS)
        eps = _get_positive(root, "rms_norm_eps")
        theta = _get_positive(root, "rope_theta")
        tied = _get_bool(root, "tie_word_embeddings", False)
        bias = _get_bool(root, "attention_bias", False)

        if root.get("head_dim") is not None:
            head_dim = _get_uint(root, "head_dim", MAX_DIM)
        else:
            if hidden % heads != 0:
                raise ConfigError("config: hidden_size is not a multiple of num_attention_heads")
            head_dim = hidden // heads
        if head_dim % 2 != 0:
            raise ConfigError("config: head_dim must be even for rotary embeddings")
        if heads % kv_heads != 0:
            raise ConfigError("config: num_attention_heads is not a multiple of num_key_value_heads")

        if "hidden_act" in root and root["hidden_act"] != "silu":
            raise ConfigError('config: only hidden_act "silu" is supported')

        eos: list[int] = []
        e = root.get("eos_token_id")
        if e is not None:
            for item in (e if isinstance(e, list) else [e]):
                if isinstance(item, bool) or not isinstance(item, int) or item < 0 or item >= vocab:
                    raise ConfigError("config: eos_token_id out of range")
                eos.append(item)
        if root.get("rope_scaling") is not None:
            raise ConfigError("config: rope_scaling is not supported")
        if root.get("use_sliding_window") is True:
            raise ConfigError("config: sliding-window attention is not supported")

        return cls(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                   num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=head_dim,
                   max_position_embeddings=max_pos, rms_norm_eps=eps, rope_theta=theta,
                   tie_word_embeddings=tied, attention_bias=bias, eos_token_ids=tuple(eos), architecture=arch)

    def to_dict(self) -> dict:
        """The config.json form of this configuration (what the folder writer stores)."""
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        d["architectures"] = [d.pop("architecture")]
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        d["hidden_act"] = "silu"
        return d
