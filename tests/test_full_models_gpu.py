"""Whole models at the benchmark set's shapes — SmolLM2-135M (30 layers), SmolLM2-360M (32 layers) and SmolLM2-1.7B
(24 layers), every layer, random weights — against the plain implementation, however the work is cut (GPU).  The tiny configurations
find faults of logic; these find what only depth and real widths show (an error that grows over 30 layers, a kernel
chosen only at these sizes)."""
import numpy as np
import pytest

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu

SHAPES = {
    "smollm2-135m": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 30, "hidden_size": 576, "num_attention_heads": 9,
                     "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1536, "vocab_size": 49152,
                     "rope_theta": 100000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192,
                     "hidden_act": "silu"},
    "smollm2-360m": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 960, "num_attention_heads": 15,
                     "num_key_value_heads": 5, "head_dim": 64, "intermediate_size": 2560, "vocab_size": 49152,
                     "rope_theta": 100000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192,
                     "hidden_act": "silu"},
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["smollm2-135m", "smollm2-360m"])
def test_whole_model_however_the_work_is_cut(shape, dtype):
    import torch
    from llmi_b200.config import parse_config
    from llmi_b200.engine.model import Model
    from llmi_b200.weights.random_weights import random_tensors
    cfg = SHAPES[shape]
    V = cfg["vocab_size"]
    arch, typed = parse_config(cfg)
    spec = arch.model_spec(typed)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(spec, 5, "cpu", store)
    w = {n: t.double().numpy() for n, t in tensors.items()}
    model = Model(spec, tensors, store, "cuda:0", config=typed)
    del tensors
    rng = np.random.default_rng(8)
    reqs = {"a": rng.integers(0, V, 70).tolist(), "b": rng.integers(0, V, 9).tolist(), "c": rng.integers(0, V, 150).tolist()}
    want = {r: list(range(max(0, len(t) - 40), len(t))) for r, t in reqs.items()}       # the head on the last 40 places only
    refs = {r: P.forward(cfg, w, t, rows=want[r]) for r, t in reqs.items()}
    del w

    def last_rows(got):
        return {r: got[r][want[r]] for r in reqs}

    cuts = {"whole": H.trace_whole(reqs), "last 32 one by one": H.trace_last_decoded(reqs, 32),
            "unequal batch": H.trace_batches(reqs, 3, {"a": 30, "b": 9, "c": 120}), "portions of 50": H.trace_portions(reqs, 50)}
    first = None
    for how, (steps, most) in cuts.items():
        got = last_rows(H.collect(steps, H.replay(model, steps, most), V))
        for r in reqs:
            assert np.isfinite(got[r]).all(), (how, r)
            assert H.rel_to_max(got[r], refs[r]) < H.TOL[dtype], (how, r)
        if dtype == "float32":                          # and in 32 bits the same bits whichever way
            if first is None:
                first = got
            else:
                for r in reqs:
                    assert np.array_equal(got[r], first[r]), (how, r)


def test_smollm2_1p7b_whole_model_in_both_types():
    """The benchmark's own shape, all 24 layers.  The weights are bf16 numbers in both runs (the 32-bit path widens them
    exactly), so that ONE pass of the plain implementation (the slow part: 1.7 G weights in float64) is the oracle of
    both types.  The 32-bit path is held to the tolerance of the tiny models.  The bf16 path is held to 3e-2 of the
    largest logit here: its activations are rounded to bf16 after every product, which adds up over 24 layers of this
    width like a random walk — against the 32-bit path on the same weights the residual stream is off by 0.6 % of its
    largest entry after the first layer and by 1.6 to 1.9 % after the last, whichever kernels run (tcgen05 or
    weight-streaming products, flash or generic attention) — so the tiny models' 1.5e-2, set for two or three layers,
    is not the measure of a fault at this depth (the 30 and 32 narrower layers above do stay inside it)."""
    import torch
    from llmi_b200.config import parse_config
    from llmi_b200.engine.model import Model
    from llmi_b200.weights.random_weights import random_tensors
    cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32,
           "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152, "rope_theta": 130000.0,
           "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"}
    V = cfg["vocab_size"]
    arch, typed = parse_config(cfg)
    spec = arch.model_spec(typed)
    tensors = random_tensors(spec, 6, "cpu", torch.bfloat16)
    rng = np.random.default_rng(9)
    reqs = {"a": rng.integers(0, V, 40).tolist(), "b": rng.integers(0, V, 3).tolist(), "c": rng.integers(0, V, 90).tolist()}
    want = {r: list(range(max(0, len(t) - 12), len(t))) for r, t in reqs.items()}
    refs = {}
    w = {n: t.double().numpy() for n, t in tensors.items()}
    for r, t in reqs.items():
        refs[r] = P.forward(cfg, w, t, rows=want[r])
    del w
    for dtype in ("bfloat16", "float32"):
        model = Model(spec, tensors, torch.bfloat16 if dtype == "bfloat16" else torch.float32, "cuda:0", config=typed)
        for how, (steps, most) in {"whole": H.trace_whole(reqs), "unequal batch, then one by one": H.trace_batches(reqs, 3, {"a": 30, "b": 3, "c": 70})}.items():
            got = H.collect(steps, H.replay(model, steps, most), V)
            for r in reqs:
                g = got[r][want[r]]
                assert np.isfinite(g).all(), (dtype, how, r)
                assert H.rel_to_max(g, refs[r]) < (H.TOL["float32"] if dtype == "float32" else 3e-2), (dtype, how, r)
        del model
        torch.cuda.empty_cache()
