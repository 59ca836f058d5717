"""Generation through the Python entry point and the command line (GPU)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_llama as P
from conftest import ROOT, TINY_CONFIGS

pytestmark = pytest.mark.gpu
STORAGE = {"float32": "F32", "bfloat16": "BF16"}
# what the tests say about recorded steps holds with the library's switches at their defaults
RECORDING = os.environ.get("LLMI_GRAPHS", "1") != "0"
DEFAULT_DECODE_PLAN = (os.environ.get("LLMI_DECODE_PLAN", "live") != "padded"
                       and os.environ.get("LLMI_DECODE_VALUE_PRODUCER", "1") != "0")


def prompts_for(name, lens, seed=21):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, TINY_CONFIGS[name]["vocab_size"], n).tolist() for n in lens]


def plain_greedy_with_margin(cfg, w, prompt, n):
    """Greedy ids from the plain implementation and the smallest top-2 logit margin on the way."""
    toks, out, margin = list(prompt), [], np.inf
    for _ in range(n):
        logits = P.forward(cfg, w, toks)[-1]
        top = np.sort(logits)[-2:]
        margin = min(margin, float(top[1] - top[0]))
        out.append(int(np.argmax(logits)))
        toks.append(out[-1])
    return out, margin


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lens,n_new", [("A", [5, 9, 17], 8), ("B", [1, 12, 30, 64], 16)])
def test_greedy_generation_matches_plain(model_dirs, name, lens, n_new, dtype):
    import llmi_b200 as L
    d = model_dirs(name, STORAGE[dtype])
    cfg, w = P.read_model(d)
    model = L.load(d, dtype)
    prompts = prompts_for(name, lens)
    got = L.generate(model, prompts, max_new=n_new, ignore_eos=True)
    for p, g in zip(prompts, got):
        ref, margin = plain_greedy_with_margin(cfg, w, p, n_new)
        if dtype == "float32" or margin > 0.05:     # a near-tie may legitimately flip under bf16 rounding
            assert g == ref
        assert len(g) == n_new


def test_stop_tokens_early_ends_and_batches_in_turn(model_dirs):
    import llmi_b200 as L
    d = model_dirs("B", "F32")
    cfg, w = P.read_model(d)
    model = L.load(d, "float32")
    prompts = prompts_for("B", [3, 20, 7, 40, 11, 2, 64])
    free = L.generate(model, prompts, max_new=12, ignore_eos=True)
    # stop ids chosen from tokens that really are generated (tests/transformer_test.cpp:393-396)
    stop = {free[0][2], free[3][5]}
    per = [12, 12, 5, 12, 1, 12, 0]
    cache = model.new_cache(64 * 4)                  # room for about three sequences: several batches, slots reused
    got, info = L.generate(model, prompts, max_new=per, stop_ids=sorted(stop), cache=cache, max_batch=3, return_details=True)
    assert info["batches"] >= 3
    for g, f, n, fin in zip(got, free, per, info["finish"]):
        cut = next((i + 1 for i, t in enumerate(f[:n]) if t in stop), n)
        assert g == f[:cut]                           # the stop token is kept; nothing after it
        assert fin == ("stop" if g and g[-1] in stop else "length")
    cache.check()
    assert not cache.slots.live
    # default stop ids come from the configuration's eos_token_id
    eos = L.generate(model, prompts[:2], max_new=12)
    for g, f in zip(eos, free[:2]):
        cut = next((i + 1 for i, t in enumerate(f) if t in cfg["eos_token_id"]), 12)
        assert g == f[:cut]


def test_sampling_is_reproducible_and_independent_of_batch_mates(model_dirs):
    import llmi_b200 as L
    d = model_dirs("B", "F32")
    model = L.load(d, "float32")
    prompts = prompts_for("B", [1, 12, 30, 64])
    sp = L.SamplingParams(temperature=0.8, top_k=50, top_p=0.95, seed=5)
    a = L.generate(model, prompts, max_new=16, ignore_eos=True, sampling=sp)
    b = L.generate(model, prompts, max_new=16, ignore_eos=True, sampling=sp)
    assert a == b
    c = L.generate(model, prompts, max_new=16, ignore_eos=True, sampling=L.SamplingParams(0.8, 50, 0.95, seed=6))
    assert a != c
    alone = L.generate(model, prompts[:1], max_new=16, ignore_eos=True, sampling=sp)
    assert alone[0] == a[0]
    # temperature 0 is greedy
    assert L.generate(model, prompts, max_new=4, ignore_eos=True, sampling=L.SamplingParams(0.0, 50, 0.5, seed=9)) == \
        L.generate(model, prompts, max_new=4, ignore_eos=True)


def test_sampled_tokens_follow_the_plain_sampler(model_dirs):
    """With the same uniform numbers the device sampler picks what the plain sampler picks."""
    import llmi_b200 as L
    from llmi_b200.sampling import UniformStream
    d = model_dirs("B", "F32")
    cfg, w = P.read_model(d)
    model = L.load(d, "float32")
    prompt = prompts_for("B", [12])[0]
    sp = L.SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=3)
    got = L.generate(model, [prompt], max_new=16, ignore_eos=True, sampling=sp)[0]
    stream = UniformStream(3, 0)
    toks = list(prompt)
    for g in got:
        logits = P.forward(cfg, w, toks)[-1]
        u = stream.next()
        p = P.sampling_probabilities(logits, 0.8)
        cum = np.cumsum(p)
        near_edge = np.min(np.abs(cum - u)) < 1e-5
        assert near_edge or P.sample(logits, 0.8, 0, 1.0, u) == g
        toks.append(g)


def test_command_line(model_dirs):
    d = model_dirs("A", "F32")
    cfg, w = P.read_model(d)
    prompt = prompts_for("A", [9])[0]
    cli = os.path.join(ROOT, "bin", "llmi-generate")
    r = subprocess.run([sys.executable, cli, d, "--ids", ",".join(map(str, prompt)), "--max-new", "8", "--ignore-eos",
                        "--json", "--dtype", "fp32"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["prompt_ids"] == prompt
    assert out["generated_ids"] == P.generate_greedy(cfg, w, prompt, 8)
    assert {"load_seconds", "generate_seconds", "weight_bytes"} <= set(out)
    r = subprocess.run([sys.executable, cli, d, "--max-new", "4"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 2 and "give --prompt or --ids" in r.stderr
    r = subprocess.run([sys.executable, cli, d, "--ids", "1,x"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 2
    r = subprocess.run([sys.executable, cli, d, "--ids", "1", "--bogus"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recorded_decode_steps_survive_other_steps_in_between(model_dirs, dtype):
    """Decode steps run as recorded graphs and, when they continue the step before, patch that step's index
    block.  Whatever happens between two of them — a prompt of another sequence through the same buffers,
    a sequence that joins, one that leaves, a slot that is freed and used again, a page boundary — the logits
    of the chosen tokens must be those of the plain implementation."""
    import llmi_b200 as L
    from llmi_b200.sampling import Sampler
    d = model_dirs("C", STORAGE[dtype])            # the long-context tiny configuration
    cfg, w = P.read_model(d)
    model = L.load(d, dtype)
    V = cfg["vocab_size"]
    cache = model.new_cache(64 * 8, n_slots=4)
    sampler = Sampler(L.SamplingParams(), model.rt)
    rng = np.random.default_rng(9)
    hist = {}

    def prefill(name, n):
        slot = cache.alloc_slot()
        toks = rng.integers(0, V, n).tolist()
        logits = model.step(cache, [L.SequenceStep(slot, toks, [n - 1])]).cpu().numpy()
        hist[name] = [slot, toks, int(np.argmax(logits[0]))]

    def decode(names):
        ids = model.step_and_choose(cache, [L.SequenceStep(hist[n][0], [hist[n][2]], [0]) for n in names], sampler).tolist()
        for n, i in zip(names, ids):
            hist[n][1].append(hist[n][2])
            hist[n][2] = int(i)

    def check(name):
        slot, toks, nxt = hist[name]
        logits = P.forward(cfg, w, toks)[-1]
        top = np.sort(logits)[-2:]
        if dtype == "float32" or top[1] - top[0] > 0.05:
            assert nxt == int(np.argmax(logits)), (name, len(toks))

    prefill("a", 60)
    for _ in range(3):
        decode(["a"])                   # continued steps (patched index block)
    prefill("b", 10)                    # another step uses the buffers in between
    decode(["a"])                       # ... so this one is planned anew; it crosses a's page boundary at 64
    decode(["a"])
    check("a")
    decode(["a", "b"])                  # b joins: another batch shape
    decode(["a", "b"])
    check("a"), check("b")
    cache.free_slot(hist.pop("a")[0])   # a leaves; its slot is used again by a longer sequence
    prefill("c", 130)
    assert hist["c"][0] != hist["b"][0]
    decode(["b", "c"])
    decode(["b", "c"])
    decode(["c", "b"])                  # the same sequences in another order: not a continuation
    decode(["c", "b"])
    check("b"), check("c")
    for n in list(hist):
        cache.free_slot(hist.pop(n)[0])
    cache.check()


WIDTH_576 = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 576, "num_attention_heads": 9,
             "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1536, "vocab_size": 49152, "rope_theta": 100000.0,
             "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "width576"])
def test_logits_of_recorded_padded_decode_steps(model_dirs, tmp_path, name, dtype):
    """The path that generation and the benchmark run — ``step_and_choose`` with recorded graphs: batches padded to a
    power of two with sequences of index -1, padded page tables, the index block patched from one step to the next —
    compared on LOGITS with the plain implementation after every step (with tied random weights greedy decoding falls
    into a fixed point, so equal tokens would say little).  The tokens fed are given, not the chosen ones, so that
    one whole-sequence pass of the plain implementation gives every step's reference.  Batch sizes that are no power
    of two (5, 3), sequences that leave one by one, pages' ends crossed while decoding."""
    import torch
    import helpers as H
    import llmi_b200 as L
    from llmi_b200.sampling import Sampler
    if name == "width576":
        d = str(tmp_path)
        L.write_random_model(d, WIDTH_576, 8, torch.float32 if dtype == "float32" else torch.bfloat16)
        prompt_lens, totals = [60, 3, 64, 127, 20], [75, 12, 70, 133, 26]
    else:
        d = model_dirs(name, STORAGE[dtype])
        ctx_len = TINY_CONFIGS[name]["max_position_embeddings"]
        prompt_lens, totals = [60, 3, 64, 120, 20], [75, 12, 70, min(128, ctx_len), 26]
    cfg, w = P.read_model(d)
    model = L.load(d, dtype)
    V = cfg["vocab_size"]
    rng = np.random.default_rng(17)
    toks = [rng.integers(0, V, n).tolist() for n in totals]
    refs = [P.forward(cfg, w, t) for t in toks]
    sampler = Sampler(L.SamplingParams(), model.rt)
    for round_ in range(2):                    # twice: the second cache replays nothing of the first one's graphs
        cache = model.new_cache(sum(H.round_up(n) for n in totals) + 64 * round_, n_slots=8)
        slots = [cache.alloc_slot() for _ in toks]
        fed = list(prompt_lens)
        model.step(cache, [L.SequenceStep(s, t[:n], []) for s, t, n in zip(slots, toks, fed)])
        live = list(range(len(toks)))
        n_steps = 0
        while live:
            ids = model.step_and_choose(cache, [L.SequenceStep(slots[i], [toks[i][fed[i]]], [0]) for i in live], sampler)
            logits = model.last_logits.cpu().numpy()
            assert logits.shape == (len(live), V)
            assert ids.tolist() == logits.argmax(1).tolist()
            for row, i in enumerate(live):
                assert np.isfinite(logits[row]).all()
                assert H.rel_to_max(logits[row], refs[i][fed[i]]) < H.TOL[dtype], (name, round_, i, fed[i])
                fed[i] += 1
            for i in [i for i in live if fed[i] == totals[i]]:
                cache.free_slot(slots[i])
                live.remove(i)
            n_steps += 1
        cache.check()
        if RECORDING:
            assert model._graphs is not None and model._graphs.replays > 0
    assert n_steps == max(t - p for t, p in zip(totals, prompt_lens))


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "width576"])
def test_logits_of_padded_and_recorded_prompt_steps(model_dirs, tmp_path, name):
    """Short prompt steps in bfloat16 are padded to a shape (token rows of no sequence up to a multiple of 64,
    sequences and wanted rows to a power of two, page tables) and a shape that comes again is recorded and replayed.
    The same batches of unequal prompts are run four times over fresh slots of one cache — plainly, plainly and
    recorded, replayed, replayed — with EVERY row's logits compared with the plain implementation each time; then the
    sequences go on in a portion of several tokens (a prompt step over a cache that is not empty) and one token at a
    time, which shows that the padding rows left nothing in the cache.  A prompt longer than the padded range (more
    than 1,024 tokens) runs beside them launch by launch."""
    import torch
    import helpers as H
    import llmi_b200 as L
    from llmi_b200.sampling import Sampler
    if name == "width576":
        d = str(tmp_path)
        L.write_random_model(d, WIDTH_576, 8, torch.bfloat16)
        batches = [[50, 3, 130], [200], [64, 64], [1100]]
        more, tail = 9, 3
    else:
        d = model_dirs(name, STORAGE["bfloat16"])
        ctx_len = TINY_CONFIGS[name]["max_position_embeddings"]
        batches = [[50, 3, min(100, ctx_len - 16)], [min(120, ctx_len - 16)], [64, 64]]
        more, tail = 9, 3
    cfg, w = P.read_model(d)
    model = L.load(d, "bfloat16")
    assert model.pads_prompts
    V = cfg["vocab_size"]
    rng = np.random.default_rng(23)
    sampler = Sampler(L.SamplingParams(), model.rt)
    cache = model.new_cache(sum(H.round_up(n + more + tail) for b in batches for n in b), n_slots=8)
    for round_ in range(4):
        for lens in batches:
            toks = [rng.integers(0, V, n + more + tail).tolist() for n in lens]
            refs = [P.forward(cfg, w, t) for t in toks]
            slots = [cache.alloc_slot() for _ in toks]
            logits = model.step(cache, [L.SequenceStep(s, t[:n], list(range(n))) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
            assert logits.shape == (sum(lens), V) and np.isfinite(logits).all()
            row = 0
            for t, n, ref in zip(toks, lens, refs):
                for i in range(n):
                    assert H.rel_to_max(logits[row + i], ref[i]) < H.TOL["bfloat16"], (name, round_, lens, i)
                row += n
            # the same sequences go on by several tokens at once (their last logits wanted), then one by one
            logits = model.step(cache, [L.SequenceStep(s, t[n:n + more], [more - 1]) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
            for r, (n, ref) in enumerate(zip(lens, refs)):
                assert H.rel_to_max(logits[r], ref[n + more - 1]) < H.TOL["bfloat16"], (name, round_, lens, "portion")
            for j in range(tail):
                model.step_and_choose(cache, [L.SequenceStep(s, [t[n + more + j]], [0]) for s, t, n in zip(slots, toks, lens)], sampler)
                logits = model.last_logits.cpu().numpy()
                for r, (n, ref) in enumerate(zip(lens, refs)):
                    assert H.rel_to_max(logits[r], ref[n + more + j]) < H.TOL["bfloat16"], (name, round_, lens, "decode", j)
            for s in slots:
                cache.free_slot(s)
            cache.check()
    g = model._prompt_graphs
    if RECORDING:
        assert g is not None and g.replays >= 2 * len([b for b in batches if sum(b) <= 1024]), (g.replays, len(g.graphs))


def test_one_model_many_caches_of_different_sizes(model_dirs):
    """A model is reused across ``generate`` calls that each make a cache of their own, of different sizes but the same
    batch and page bucket: a recorded step must never be replayed against another cache's memory."""
    import gc
    import llmi_b200 as L
    d = model_dirs("C", "F32")
    cfg, w = P.read_model(d)
    model = L.load(d, "float32")
    prompts = prompts_for("C", [30, 5, 17])
    ref = [P.generate_greedy(cfg, w, p, 40) for p in prompts]
    for max_new in (9, 40, 23, 33, 12):
        got = L.generate(model, prompts, max_new=max_new, ignore_eos=True)
        assert got == [r[:max_new] for r in ref], max_new
        gc.collect()
        serials = {k[3] for k in model._graphs.graphs}
        assert len(serials) <= 1, "graphs of dead caches must be dropped"


MANY_HEADS = {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 1, "hidden_size": 128, "num_attention_heads": 32,
              "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 192, "vocab_size": 320, "rope_theta": 10000.0,
              "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 1024, "hidden_act": "silu"}


def test_recorded_decode_steps_of_one_shape_are_told_apart_by_their_plan(tmp_path):
    """16, then 9, then 2 live sequences: the first two are padded to the same shape (16), but their decode kernels
    are cut into items differently (9 x 32 sequence-heads fit the variant with whole sequence-heads as items, 16 x 32
    do not), so they are recorded apart; the 2 run the kernel's cluster form; every step's logits are the plain
    implementation's."""
    import torch
    import helpers as H
    import llmi_b200 as L
    from llmi_b200.ops import kernels
    from llmi_b200.sampling import Sampler
    d = str(tmp_path)
    L.write_random_model(d, MANY_HEADS, 3, torch.bfloat16)
    cfg, w = P.read_model(d)
    model = L.load(d, "bfloat16")
    V = cfg["vocab_size"]
    rng = np.random.default_rng(5)
    n_seqs, prompt, steps = 16, 250, 9          # the decode steps cross a page's end (256)
    toks = [rng.integers(0, V, prompt + steps).tolist() for _ in range(n_seqs)]
    refs = [P.forward(cfg, w, t) for t in toks]
    sampler = Sampler(L.SamplingParams(), model.rt)
    cache = model.new_cache(n_seqs * 320, n_slots=16)
    slots = [cache.alloc_slot() for _ in toks]
    model.step(cache, [L.SequenceStep(s, t[:prompt], []) for s, t in zip(slots, toks)])
    live, fed, tokens_seen = list(range(n_seqs)), prompt, set()
    for step in range(steps):
        if step == 3:
            for i in live[9:]:
                cache.free_slot(slots[i])
            live = live[:9]
        if step == 6:
            for i in live[2:]:
                cache.free_slot(slots[i])
            live = live[:2]
        model.step_and_choose(cache, [L.SequenceStep(slots[i], [toks[i][fed]], [0]) for i in live], sampler)
        logits = model.last_logits.cpu().numpy()
        for row, i in enumerate(live):
            assert H.rel_to_max(logits[row], refs[i][fed]) < H.TOL["bfloat16"], (step, i)
        fed += 1
        tokens_seen.add((len(live), model.step_plan_token(model._graphs._last[2], cache)))
    cache.check()
    if RECORDING and DEFAULT_DECODE_PLAN:
        plans = {n: t for n, t in tokens_seen}
        assert len(tokens_seen) == 3 and plans[16] != plans[9], plans       # 16 and 9 share a padded shape, not a plan
        keys = [k for k in model._graphs.graphs if k[0] == 16]
        assert len({k[-1] for k in keys}) == 2, keys
        assert model._graphs.replays >= 3
        if os.environ.get("LLMI_DECODE_CLUSTER", "1") != "0" and kernels.sm_count() >= 132:
            assert plans[2][0][2] in (2, 4), plans      # 2 x 32 sequence-heads of 5 pages: the kernel's cluster form
