"""The kernels that only large shapes reach — the product on pairs of SMs (256 tokens and more), the cluster
k-split (17 to about 1,000 tokens), the tcgen05 prompt attention (head sizes 64 and 128), the tensor-core decode
attention for grouped queries — inside the model: two layers at SmolLM2-1.7B width, and two at the width of an
8B Llama (4,096 wide, 32 heads of 128 over 8 kv heads, feed-forward 14,336), the bf16 path against the 32-bit
path of the same seeded weights (GPU)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CONFIG = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 2048, "num_attention_heads": 32,
          "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152, "rope_theta": 130000.0,
          "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"}


WIDE = dict(CONFIG, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=14336,
            vocab_size=32000, rope_theta=500000.0, tie_word_embeddings=False)


def run(model, prompts, n_decode, seed, V=CONFIG["vocab_size"]):
    import llmi_b200 as L
    rng = np.random.default_rng(seed)
    cache = model.new_cache(sum((len(p) + n_decode + 63) // 64 * 64 for p in prompts), n_slots=len(prompts))
    slots = [cache.alloc_slot() for _ in prompts]
    out = [model.step(cache, [L.SequenceStep(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)]).float().cpu().numpy().copy()]
    for _ in range(n_decode):
        toks = [int(t) for t in rng.integers(0, V, len(prompts))]
        out.append(model.step(cache, [L.SequenceStep(s, [t], [0]) for s, t in zip(slots, toks)]).float().cpu().numpy().copy())
    return out


@pytest.mark.parametrize("lens,n_decode", [([1, 63, 64, 65, 1000, 3000], 3), ([int(n) for n in range(100, 380, 4)], 2)],
                         ids=["ragged-to-3000", "70-sequences"])
def test_bf16_path_follows_the_32_bit_path_at_full_width(lens, n_decode):
    import llmi_b200 as L
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(1)
    prompts = [rng.integers(0, CONFIG["vocab_size"], n).tolist() for n in lens]
    fast = run(L.random_model(CONFIG, seed=3, dtype="bfloat16", on_device=True), prompts, n_decode, 5)
    exact = run(L.random_model(CONFIG, seed=3, dtype="float32", on_device=True), prompts, n_decode, 5)
    kernels.check_device_errors("cuda:0")
    for a, b in zip(fast, exact):
        assert np.isfinite(a).all()
        # the bf16 model's weights are the rounded 32-bit ones: about 1.3 % of the largest logit in practice
        assert float(np.abs(a - b).max() / np.abs(b).max()) < 3e-2


def test_bf16_path_follows_the_32_bit_path_at_8b_width():
    import llmi_b200 as L
    from llmi_b200.ops import kernels
    rng = np.random.default_rng(2)
    V = WIDE["vocab_size"]
    prompts = [rng.integers(0, V, n).tolist() for n in (1, 70, 129, 300, 700)]
    fast = run(L.random_model(WIDE, seed=4, dtype="bfloat16", on_device=True), prompts, 3, 6, V)
    exact = run(L.random_model(WIDE, seed=4, dtype="float32", on_device=True), prompts, 3, 6, V)
    kernels.check_device_errors("cuda:0")
    for a, b in zip(fast, exact):
        assert np.isfinite(a).all()
        assert float(np.abs(a - b).max() / np.abs(b).max()) < 3e-2
