"""The kernels that only large shapes reach — the product on pairs of SMs (256 tokens and more), the cluster
k-split (17 to about 1,000 tokens), the tcgen05 prompt attention (head sizes 64 and 128), the tensor-core decode
attention for grouped queries — inside the model: two layers at SmolLM2-1.7B width, and two at the width of an
8B Llama (4,096 wide, 32 heads of 128 over 8 kv heads, feed-forward 14,336): both paths against the plain
implementation on a few hundred tokens, and the bf16 path against the 32-bit path of the same seeded weights on
thousands (GPU)."""
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ["width-2048", "width-4096"])
def test_full_width_layers_follow_the_plain_implementation(shape, dtype):
    """The oracle for the kernels the benchmark consists of is the plain implementation, not the engine's other path:
    two layers at full width, prompts of a few hundred tokens in one step (more than 512 tokens at width 2,048, so
    that the product runs on pairs of SMs; 129 to 511 at width 4,096, where its k range is cut over a cluster; the
    tcgen05 prompt attention at both head sizes), then decode steps through the recorded-graph path."""
    import torch
    import helpers as H
    import plain_llama as P
    import llmi_b200 as L
    from llmi_b200.config import parse_config
    from llmi_b200.engine.model import Model
    from llmi_b200.sampling import Sampler
    from llmi_b200.weights.random_weights import random_tensors
    cfg = dict(CONFIG) if shape == "width-2048" else dict(WIDE, vocab_size=8000)
    lens = [400, 130, 1] if shape == "width-2048" else [300, 60]
    n_decode = 3
    V = cfg["vocab_size"]
    arch, typed = parse_config(cfg)
    spec = arch.model_spec(typed)
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = random_tensors(spec, 21, "cpu", store)
    w = {n: t.double().numpy() for n, t in tensors.items()}
    model = Model(spec, tensors, store, "cuda:0", config=typed)
    del tensors
    rng = np.random.default_rng(4)
    toks = [rng.integers(0, V, n + n_decode).tolist() for n in lens]
    refs = [P.forward(cfg, w, t, rows=list(range(n - 1, n + n_decode))) for t, n in zip(toks, lens)]
    del w
    cache = model.new_cache(sum(H.round_up(len(t)) for t in toks), n_slots=len(toks))
    slots = [cache.alloc_slot() for _ in toks]
    got = [[] for _ in toks]
    out = model.step(cache, [L.SequenceStep(s, t[:n], [n - 1]) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
    for i in range(len(toks)):
        got[i].append(out[i].copy())
    sampler = Sampler(L.SamplingParams(), model.rt)
    for j in range(n_decode):
        model.step_and_choose(cache, [L.SequenceStep(s, [t[n + j]], [0]) for s, t, n in zip(slots, toks, lens)], sampler)
        out = model.last_logits.cpu().numpy()
        for i in range(len(toks)):
            got[i].append(out[i].copy())
    from llmi_b200.ops import kernels
    kernels.check_device_errors("cuda:0")
    for i in range(len(toks)):
        g = np.stack(got[i])
        assert np.isfinite(g).all()
        assert H.rel_to_max(g, refs[i]) < H.TOL[dtype], (shape, dtype, i)


@pytest.mark.parametrize("config", [CONFIG, WIDE], ids=["width-2048", "width-4096-heads-of-128"])
def test_the_same_step_again_and_again_gives_the_same_bits(config):
    """Steps of full-width layers run repeatedly on the same context — a long prompt, unequal prompts, decode steps at
    batch sizes that reach every product kernel — must give the bits of the first run every time: a race between a
    copy engine and the threads, or a wait that passes a phase too early, shows as a result that differs now and then
    (two such faults were found this way), long before it is large enough to fail a comparison with a tolerance."""
    import torch
    import llmi_b200 as L
    from llmi_b200.engine.batch import plan_step
    from llmi_b200.ops import kernels
    model = L.random_model(dict(config, num_hidden_layers=2), seed=4, dtype="bfloat16", on_device=True)
    V = config["vocab_size"]
    rng = np.random.default_rng(2)
    for what, lens, reps in (("prompt", [2048], 8), ("prompt", [300, 40, 1000], 8), ("prompt", [17], 12), ("decode", [500] * 16, 20),
                             ("decode", [700] * 40, 20), ("decode", [3000] * 8, 20)):
        cache = model.new_cache(sum((n + 1 + 63) // 64 * 64 for n in lens) + 64, n_slots=64)
        slots = [cache.alloc_slot() for _ in lens]
        toks = [rng.integers(0, V, n + 1).tolist() for n in lens]
        if what == "decode":
            for s, t, n in zip(slots, toks, lens):
                model.step(cache, [L.SequenceStep(s, t[:n], [])])
            ctx = plan_step(cache, [L.SequenceStep(s, [t[n]], [0]) for s, t, n in zip(slots, toks, lens)], V, model.buffers)
        else:
            ctx = plan_step(cache, [L.SequenceStep(s, t[:n], [n - 1, n // 2]) for s, t, n in zip(slots, toks, lens)], V, model.buffers)
        first = model.run(ctx, cache).clone()
        assert torch.isfinite(first).all()
        for _ in range(reps):
            assert torch.equal(model.run(ctx, cache), first), (what, lens)
        kernels.check_device_errors("cuda:0")
        del cache
