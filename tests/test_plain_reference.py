"""The plain implementation against the reference engine's own binary (stored outputs)."""
import os

import numpy as np
import pytest

import plain_llama as P
from golden import make_golden as G

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_tiny.npz"))


def rel(a, b):
    return float(np.max(np.abs(a - b)) / np.max(np.abs(b)))


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_and_states_match_reference_binary(tmp_path, name):
    G.write_model(str(tmp_path), name)
    cfg, w = P.read_model(str(tmp_path))
    logits, states = P.forward(cfg, w, G.PROMPTS[name], return_states=True)
    ref_states = GOLD[f"{name}_states"]
    assert len(states) == ref_states.shape[0] == cfg["num_hidden_layers"] + 2
    for s, r in zip(states, ref_states):
        assert rel(s, r) < 2e-6
    assert rel(logits, GOLD[f"{name}_logits"]) < 2e-6
    assert (np.argmax(logits, 1) == np.argmax(GOLD[f"{name}_logits"], 1)).all()


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_arithmetic_matches_too(tmp_path, name):
    G.write_model(str(tmp_path), name)
    cfg, w = P.read_model(str(tmp_path))
    logits = P.forward(cfg, w, G.PROMPTS[name], dtype=np.float32)
    assert rel(logits, GOLD[f"{name}_logits"]) < 1e-4     # the reference's own tolerance (ADR 0003)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_matches_reference_binary(tmp_path, name):
    G.write_model(str(tmp_path), name)
    cfg, w = P.read_model(str(tmp_path))
    out = P.generate_greedy(cfg, w, G.PROMPTS[name], 8)
    assert out == GOLD[f"{name}_greedy"].tolist() == GOLD[f"{name}_greedy_cached"].tolist()


def test_planted_faults_are_seen(tmp_path):
    """The comparison has teeth: each of the classic faults moves the logits far beyond tolerance
    (the reference's own planted-bug study: docs/forward-pass.md:41-56)."""
    G.write_model(str(tmp_path), "A")
    cfg, w = P.read_model(str(tmp_path))
    good = GOLD["A_logits"]
    ids = G.PROMPTS["A"]

    bad_theta = dict(cfg, rope_theta=500.0)
    assert rel(P.forward(bad_theta, w, ids), good) > 1e-3

    orig = P.attention
    try:
        def wrong_group(q, k, v, window=0):        # h % nkv instead of h // group
            T, nh, d = q.shape
            out = np.zeros_like(q)
            for hh in range(nh):
                kvh = hh % k.shape[1]
                for t in range(T):
                    p = P.softmax((k[:t + 1, kvh] @ q[t, hh]) / np.sqrt(d))
                    out[t, hh] = p @ v[:t + 1, kvh]
            return out
        P.attention = wrong_group
        assert rel(P.forward(cfg, w, ids), good) > 1e-3
    finally:
        P.attention = orig

    orig_rope = P.rope
    try:
        def interleaved(v, positions, inv_freq):   # pairs (2i, 2i+1) instead of (i, i + d/2)
            angle = np.asarray(positions, dtype=np.float64)[:, None] * inv_freq[None, :]
            c, s = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
            a, b = v[..., 0::2], v[..., 1::2]
            out = np.empty_like(v)
            out[..., 0::2], out[..., 1::2] = a * c - b * s, b * c + a * s
            return out
        P.rope = interleaved
        assert rel(P.forward(cfg, w, ids), good) > 1e-3
    finally:
        P.rope = orig_rope


def test_parts_alone():
    x = np.array([[3.0, 4.0]])
    y = P.rmsnorm(x, np.array([1.0, 2.0]), 0.0)
    assert np.allclose(y, [[3 / np.sqrt(12.5), 8 / np.sqrt(12.5)]])
    inv = P.rope_inv_freq(4, 10000.0)
    v = np.arange(8, dtype=np.float64).reshape(1, 2, 4)
    assert np.allclose(P.rope(v, [0], inv), v)                       # position 0 is the identity
    r = P.rope(v, [3], inv)
    assert np.allclose(np.linalg.norm(r, axis=-1), np.linalg.norm(v, axis=-1))
    assert abs(P.silu(0.0)) == 0 and np.isclose(P.silu(1.0), 1 / (1 + np.exp(-1)))
    assert P.argmax(np.array([1.0, 5.0, 5.0])) == 1
    p = P.sampling_probabilities(np.array([0.0, 1.0, 2.0, 3.0]), 1.0, top_k=2)
    assert np.count_nonzero(p) == 2 and np.isclose(p.sum(), 1.0)
    p = P.sampling_probabilities(np.array([0.0, 0.0, 10.0]), 1.0, top_p=0.5)
    assert np.count_nonzero(p) == 1


@pytest.mark.parametrize("rows", ["A", "B", "ties"])
def test_sampling_probabilities_match_the_reference_library(rows):
    """The distribution the sampler draws from (src/model/sampling.cpp:11-58), recorded from the reference's own
    library for real and made-up rows of logits, exact ties included: the same tokens survive top-k and top-p, and
    their probabilities agree to float rounding."""
    logits = GOLD[f"sampling_{rows}_logits"]
    for i, (temperature, top_k, top_p) in enumerate(G.SAMPLING):
        ref = GOLD[f"sampling_{rows}_{i}"]
        for r in range(logits.shape[0]):
            p = P.sampling_probabilities(logits[r], temperature, top_k, top_p)
            assert np.array_equal(p > 0, ref[r] > 0), (rows, i, r)
            assert np.allclose(p, ref[r], rtol=2e-6, atol=1e-12), (rows, i, r)
            assert abs(ref[r].sum() - 1.0) < 1e-5


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_sequence_continued_in_portions_is_the_whole_sequence(tmp_path, name):
    """The reference's ``forward_cached`` fed in portions of several tokens gives its whole-sequence logits bit for bit
    (include/llmi/model/transformer.hpp:25-28), so the plain whole-sequence pass is the oracle for portions too."""
    assert np.array_equal(GOLD[f"{name}_portions_logits"], GOLD[f"{name}_logits"])
    G.write_model(str(tmp_path), name)
    cfg, w = P.read_model(str(tmp_path))
    assert rel(P.forward(cfg, w, G.PROMPTS[name]), GOLD[f"{name}_portions_logits"]) < 2e-6
