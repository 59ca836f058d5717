"""Random tiny configurations (head sizes in steps of 16, groups, widths and vocabularies that are no power of two,
with and without q/k/v biases and a tied head) and random traces — up to three live requests that start with prompts
or portions of them, go on by 1, 2, 7, 63, 64, 65, 100 or 300 tokens or by one token each, end at different times and
leave their slots to the next — against the plain implementation, in both types, over a cache whose pages start out
as NaN.  Each trace runs three times over, so that in bfloat16 the padded prompt steps come again, are recorded and
replayed (GPU)."""
import os

import numpy as np
import pytest

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu


def random_config(rng):
    hd = int(rng.choice([16, 32, 48, 64, 128]))
    nkv = int(rng.choice([1, 2, 3]))
    nh = nkv * int(rng.choice([1, 2, 3, 4]))
    return {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": int(rng.integers(1, 4)),
            "hidden_size": int(rng.choice([nh * hd, 8 * int(rng.integers(5, 40))])), "num_attention_heads": nh,
            "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": 8 * int(rng.integers(4, 60)),
            "vocab_size": int(rng.integers(40, 700)), "rope_theta": float(rng.choice([10000.0, 130000.0])),
            "rms_norm_eps": float(rng.choice([1e-5, 1e-6])), "tie_word_embeddings": bool(rng.integers(0, 2)),
            "max_position_embeddings": 1024, "hidden_act": "silu", "attention_bias": bool(rng.integers(0, 2))}


def random_trace(rng, reqs):
    """Steps as the trace replayer reads them; every entry also says where its tokens start in the request (``at``)."""
    steps, fed, live, waiting, k = [], {}, [], list(reqs), 0
    while live or waiting:
        while waiting and len(live) < 3 and (not live or rng.random() < 0.5):
            r = waiting.pop(0)
            live.append(r)
            fed[r] = 0
        decode_step = rng.random() < 0.6
        entries = []
        for r in live:
            left = len(reqs[r]) - fed[r]
            n = 1 if (fed[r] > 0 and decode_step) else int(rng.choice([1, 2, 7, 63, 64, 65, 100, 300]))
            n = max(1, min(n, left))
            want = sorted({n - 1, *(int(x) for x in rng.integers(0, n, min(n, 3)))})
            entries.append({"id": r, "tokens": reqs[r][fed[r]:fed[r] + n], "want": want, "at": fed[r]})
            fed[r] += n
        ending = [r for r in live if fed[r] == len(reqs[r])]
        steps.append({"step": k, "entries": entries, "end": ending})
        k += 1
        live = [r for r in live if r not in ending]
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [21, 22, 23, 24, 25])
def test_random_configuration_and_trace(tmp_path, seed, dtype):
    import torch
    import llmi_b200 as L
    from llmi_b200.engine.trace import TraceReplayer
    rng = np.random.default_rng(seed)
    cfg = random_config(rng)
    L.write_random_model(str(tmp_path), cfg, seed, torch.float32 if dtype == "float32" else torch.bfloat16)
    c, w = P.read_model(str(tmp_path))
    model = L.load(str(tmp_path), dtype)
    V = cfg["vocab_size"]
    lengths = [int(rng.choice([rng.integers(2, 40), rng.integers(40, 200), rng.integers(200, 520)])) for _ in range(int(rng.integers(3, 8)))]
    reqs = {f"r{i}": rng.integers(0, V, n).tolist() for i, n in enumerate(lengths)}
    refs = {r: P.forward(c, w, t) for r, t in reqs.items()}
    steps = random_trace(rng, reqs)
    rp = TraceReplayer(model, 3 * 576)
    for g in rp.cache.kv_groups:
        g.k.fill_(float("nan"))
        g.v.fill_(float("nan"))
    for round_ in range(3):
        for s in steps:
            out = rp.run_step(s)
            off = 0
            for e in s["entries"]:
                for place in e["want"]:
                    assert np.isfinite(out[off]).all(), (cfg, round_, s["step"], e["id"])
                    assert H.rel_to_max(out[off], refs[e["id"]][e["at"] + place]) < H.TOL[dtype], (cfg, round_, s["step"], e["id"], e["at"] + place)
                    off += 1
            assert off == out.shape[0]
        rp.cache.check()
        assert not rp.slots
    if dtype == "bfloat16" and model.pads_prompts and os.environ.get("LLMI_GRAPHS", "1") != "0":
        assert model._prompt_graphs is not None and model._prompt_graphs.replays > 0
