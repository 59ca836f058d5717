"""The engine against the plain implementation, however the work is cut (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers as H
import plain_llama as P
from conftest import ROOT, TINY_CONFIGS

pytestmark = pytest.mark.gpu

STORAGE = {"float32": "F32", "bfloat16": "BF16"}
CONFIG_NAMES = ["A", "B", "C", "D"]
LENGTHS = {"A": [5, 9, 17, 40, 100, 128], "B": [1, 12, 30, 64, 65, 200], "C": [3, 33, 64, 129, 300, 700],
           "D": [2, 31, 64, 66, 150, 199]}


def make_requests(name, seed=11):
    rng = np.random.default_rng(seed)
    v = TINY_CONFIGS[name]["vocab_size"]
    return {f"r{i}": rng.integers(0, v, n).tolist() for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def loaded(model_dirs):
    import llmi_b200 as L
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            d = model_dirs(name, STORAGE[dtype])
            cfg, w = P.read_model(d)
            reqs = make_requests(name)
            refs = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
            cache[(name, dtype)] = (L.load(d, dtype), reqs, refs, d)
        return cache[(name, dtype)]
    return get


def check(got, refs, dtype):
    assert set(got) == set(refs)
    for r in refs:
        assert got[r].shape == refs[r].shape
        assert np.isfinite(got[r]).all(), f"{r}: non-finite logits (something outside the sequence was read)"
        assert H.rel_to_max(got[r], refs[r]) < H.TOL[dtype], r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_whole_requests(loaded, name, dtype):
    model, reqs, refs, _ = loaded(name, dtype)
    steps, most = H.trace_whole(reqs)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", ["A", "B"])
def test_f16_weights_are_used_exactly_in_the_32_bit_path(model_dirs, name):
    """A folder stored as F16 and run in fp32 computes with the file's values (src/model/safetensors.cpp:290-299 widens
    each element exactly): all three ways of cutting match the plain implementation, which reads F16 exactly, at the
    32-bit tolerance.  (Rounding the weights to bf16 on the way would miss it by two orders of magnitude.)"""
    import llmi_b200 as L
    d = model_dirs(name, "F16")
    cfg, w = P.read_model(d)
    model = L.load(d, "float32")
    reqs = make_requests(name)
    refs = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
    rng = np.random.default_rng(3)
    prompt_lens = {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()}
    for steps, most in (H.trace_whole(reqs), H.trace_last_decoded(reqs, 32), H.trace_batches(reqs, 3, prompt_lens)):
        check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, "float32")
    # and in bf16 the one rounding is that of the compute type
    fast = L.load(d, "bfloat16")
    steps, most = H.trace_whole(reqs)
    check(H.collect(steps, H.replay(fast, steps, most), fast.vocab_size), refs, "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_last_32_tokens_one_by_one(loaded, name, dtype):
    model, reqs, refs, _ = loaded(name, dtype)
    steps, most = H.trace_last_decoded(reqs, 32)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_unequal_batches_one_after_another(loaded, name, dtype):
    model, reqs, refs, _ = loaded(name, dtype)
    rng = np.random.default_rng(3)
    prompt_lens = {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()}
    prompt_lens["r0"] = len(reqs["r0"])            # one request is all prompt and ends at once
    steps, most = H.trace_batches(reqs, 3, prompt_lens)
    # the cache is sized for one batch: the second batch can only run in the first one's slots and pages
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(loaded, dtype):
    """A one-token prompt followed by hundreds of single-token steps: the first tokens of a sequence
    (positions 0, 1, 2 with one, two, three keys) and decoding across many page borders."""
    model, reqs, refs, _ = loaded("C", dtype)
    toks = reqs["r5"]
    steps, most = H.trace_last_decoded({"r5": toks}, n_last=len(toks) - 1)
    got = H.collect(steps, H.replay(model, steps, most), model.vocab_size)
    check(got, {"r5": refs["r5"]}, dtype)
    assert H.rel_to_max(got["r5"][:3], refs["r5"][:3]) < H.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("portion", [7, 64, 100])
@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_prompt_in_portions(loaded, name, portion, dtype):
    """A prompt fed in portions, then decoded: every portion but the first continues a sequence by more than one
    token (include/llmi/model/transformer.hpp:89-95), across page ends (64) and inside pages (7, 100)."""
    model, reqs, refs, _ = loaded(name, dtype)
    steps, most = H.trace_portions(reqs, portion)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_portions_beside_decoding_sequences(loaded, name, dtype):
    """One batch whose steps mix sequences that continue their prompt by several tokens with sequences that decode."""
    model, reqs, refs, _ = loaded(name, dtype)
    ids = list(reqs)
    first = {r: max(1, len(reqs[r]) // 3) for r in ids}
    portion = {r: (1, 2, 63, 1, 65, 5)[i % 6] for i, r in enumerate(ids)}
    steps, most = H.trace_mixed(reqs, first, portion)
    assert any(len({len(e["tokens"]) for e in s["entries"]}) > 1 and s["step"] > 0 for s in steps)
    check(H.collect(steps, H.replay(model, steps, most), model.vocab_size), refs, dtype)


@pytest.mark.parametrize("name", CONFIG_NAMES)
def test_cutting_does_not_change_fp32_logits_at_all(loaded, name):
    """In the 32-bit path every reduction runs in an order that depends on absolute positions only, so the logits of a
    position are the same BITS whole, token by token, in portions and in unequal batches — the reference's own claim
    for its cache (include/llmi/model/transformer.hpp:25-28; tests/transformer_test.cpp:322-411)."""
    model, reqs, refs, _ = loaded(name, "float32")
    V = model.vocab_size
    s1, m1 = H.trace_whole(reqs)
    whole = H.collect(s1, H.replay(model, s1, m1), V)
    rng = np.random.default_rng(3)
    prompt_lens = {r: int(rng.integers(1, len(t) + 1)) for r, t in reqs.items()}
    ids = list(reqs)
    cuts = {
        "last 32 one by one": H.trace_last_decoded(reqs, 32),
        "unequal batches": H.trace_batches(reqs, 3, prompt_lens),
        "portions of 1": H.trace_portions(reqs, 1),
        "portions of 2": H.trace_portions(reqs, 2),
        "portions of 63": H.trace_portions(reqs, 63),
        "portions of 64": H.trace_portions(reqs, 64),
        "portions of 65": H.trace_portions(reqs, 65),
        "mixed": H.trace_mixed(reqs, {r: max(1, len(reqs[r]) // 2) for r in ids},
                               {r: (1, 3, 64)[i % 3] for i, r in enumerate(ids)}),
    }
    for how, (steps, most) in cuts.items():
        got = H.collect(steps, H.replay(model, steps, most), V)
        for r in reqs:
            assert np.array_equal(got[r], whole[r]), (how, r)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(loaded, tmp_path, dtype):
    """bin/trace_run as a user calls it: a subprocess, steps on standard input, files out."""
    model, reqs, refs, d = loaded("A", dtype)
    sub = {r: reqs[r] for r in ("r1", "r2", "r3")}
    steps, most = H.trace_batches(sub, 3, {"r1": 4, "r2": 17, "r3": 9})
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(most)],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outs = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        outs.append(np.fromfile(f, dtype="<f4").reshape(n, -1) if n else None)
        assert f.exists() == bool(n)
    check(H.collect(steps, outs, model.vocab_size), {r: refs[r] for r in sub}, dtype)


def test_step_errors(loaded):
    import llmi_b200 as L
    from llmi_b200.cache import CacheError
    model, reqs, _, _ = loaded("A", "float32")
    cache = model.new_cache(128)
    s = cache.alloc_slot()
    with pytest.raises(L.StepError, match="out of range"):
        model.step(cache, [L.SequenceStep(s, [model.vocab_size], [0])])
    with pytest.raises(L.StepError, match="no tokens"):
        model.step(cache, [L.SequenceStep(s, [], [])])
    with pytest.raises(L.StepError, match="twice"):
        model.step(cache, [L.SequenceStep(s, [1], [0]), L.SequenceStep(s, [2], [0])])
    with pytest.raises(CacheError, match="not live"):
        model.step(cache, [L.SequenceStep(s + 1, [1], [0])])
    with pytest.raises(CacheError, match="context"):
        model.step(cache, [L.SequenceStep(s, [1] * 129, [0])])
    s2 = cache.alloc_slot()
    model.step(cache, [L.SequenceStep(s, [1] * 64, [63])])
    with pytest.raises(CacheError, match="full"):
        model.step(cache, [L.SequenceStep(s2, [1] * 65, [0])])
    assert cache.length(s2) == 0                       # a refused step reserves nothing
    model.step(cache, [L.SequenceStep(s2, [1] * 64, [0])])
    cache.free_slot(s2)
    model.step(cache, [L.SequenceStep(s, [1, 2], [0])])        # a sequence may go on by more than one token
    assert cache.length(s) == 66
    s2 = cache.alloc_slot()
    other = model.new_cache(64)
    with pytest.raises(ValueError, match="not created"):
        L.load(loaded("A", "float32")[3], "float32").step(other, [L.SequenceStep(0, [1], [0])])
    cache.free_slot(s)
    cache.free_slot(s2)
    cache.check()


def test_causality(loaded):
    """Changing a later token leaves the logits of earlier positions bit-identical
    (tests/transformer_test.cpp:201-218)."""
    import llmi_b200 as L
    model, reqs, _, _ = loaded("A", "float32")
    cache = model.new_cache(128)
    toks = list(reqs["r2"])
    outs = []
    for variant in (toks, toks[:9] + [(toks[9] + 1) % 256] + toks[10:]):
        s = cache.alloc_slot()
        outs.append(model.step(cache, [L.SequenceStep(s, variant, list(range(len(variant))))]).cpu().numpy().copy())
        cache.free_slot(s)
    assert (outs[0][:9] == outs[1][:9]).all()
    assert not (outs[0][9:] == outs[1][9:]).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(576, 9, 3, 64, 1536), (320, 14, 2, 128, 520)])
def test_smollm2_135m_layer_sizes(tmp_path, dtype, sizes):
    """Two layers at SmolLM2-135M sizes (9 heads over 3 kv heads of 64, width 576, vocabulary 49,152), and two
    with 14 heads over 2 kv heads of 128: the kernels' fast paths for real head shapes (groups of 3 and 7,
    a vocabulary that is no power of two) against the plain implementation, prompt whole and then decoded."""
    import torch
    import llmi_b200 as L
    width, nh, nkv, hd, ffn = sizes
    cfg = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": width, "num_attention_heads": nh,
           "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": ffn, "vocab_size": 49152, "rope_theta": 100000.0,
           "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu",
           "eos_token_id": 0}
    L.write_random_model(str(tmp_path), cfg, 8, torch.float32 if dtype == "float32" else torch.bfloat16)
    pcfg, w = P.read_model(str(tmp_path))
    model = L.load(str(tmp_path), dtype)
    rng = np.random.default_rng(9)
    reqs = {"x": rng.integers(0, 49152, 150).tolist(), "y": rng.integers(0, 49152, 70).tolist()}
    refs = {r: P.forward(pcfg, w, t) for r, t in reqs.items()}
    steps, most = H.trace_batches(reqs, 2, {"x": 130, "y": 40})
    got = H.collect(steps, H.replay(model, steps, most), 49152)
    check(got, refs, dtype)
    for r in reqs:
        assert (got[r].argmax(1) == refs[r].argmax(1)).mean() > (0.999 if dtype == "float32" else 0.9)
