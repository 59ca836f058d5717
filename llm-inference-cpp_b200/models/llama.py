"""The Llama / SmolLM2 dense decoder as a recipe of parts.

Layer order and tensor names follow the reference (include/llmi/model/transformer.hpp:49-52;
src/model/model.cpp:135-162): token embedding; per layer RMSNorm → grouped-query attention
with rotate-half positions → residual, RMSNorm → SwiGLU → residual; final RMSNorm; a head
that is the embedding table when ``tie_word_embeddings`` is set.  Extra tensors that
exporters add are tolerated as the reference tolerates them (src/model/model.cpp:190-196).
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import Architecture, register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def llama_model_spec(c: LlamaConfig) -> ModelSpec:
    position = PartSpec("rotary_half", {"head_dim": c.head_dim, "theta": c.rope_theta})
    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        layers.append(LayerSpec(
            block="prenorm",
            mixer_norm=PartSpec("rms", {"width": c.hidden_size, "eps": c.rms_norm_eps}, p + "input_layernorm."),
            mixer=PartSpec("gqa", {"width": c.hidden_size, "n_heads": c.num_attention_heads,
                                   "n_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                                   "bias": c.attention_bias, "window": 0, "position": position},
                           p + "self_attn."),
            ffn_norm=PartSpec("rms", {"width": c.hidden_size, "eps": c.rms_norm_eps}, p + "post_attention_layernorm."),
            ffn=PartSpec("swiglu", {"width": c.hidden_size, "inner": c.intermediate_size}, p + "mlp."),
        ))
    return ModelSpec(
        architecture=c.architecture,
        vocab_size=c.vocab_size, width=c.hidden_size, max_positions=c.max_position_embeddings,
        embedding=PartSpec("token_table", {"vocab": c.vocab_size, "width": c.hidden_size}, "model.embed_tokens."),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
        final_norm=PartSpec("rms", {"width": c.hidden_size, "eps": c.rms_norm_eps}, "model.norm."),
        head=PartSpec("linear_head", {"vocab": c.vocab_size, "width": c.hidden_size, "tied": c.tie_word_embeddings},
                      "lm_head."),
        stop_ids=tuple(c.eos_token_ids),
    )


def _tolerated(name: str) -> bool:
    return name == "lm_head.weight" or "rotary_emb.inv_freq" in name


register_architecture(Architecture("LlamaForCausalLM", LlamaConfig.from_dict, llama_model_spec, _tolerated))
