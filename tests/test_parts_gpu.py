"""Each part alone, a schedule that is not the plain one, and a toy mixer with state of its own that
is registered, built and stepped without touching the library's files (GPU)."""
import numpy as np
import pytest
import torch

import helpers as H
import plain_llama as P

pytestmark = pytest.mark.gpu


def rt(dtype=torch.float32):
    from llmi_b200.engine.runtime import Runtime
    return Runtime(dtype, "cuda:0")


def spec(kind, params, prefix=""):
    from llmi_b200.parts import PartSpec
    return PartSpec(kind, params, prefix)


def test_norm_part():
    from llmi_b200.parts import get_part
    w = 1 + 0.1 * torch.randn(40)
    part = get_part("norm", "rms")(spec("rms", {"width": 40, "eps": 1e-3}), {"weight": w.to(torch.bfloat16)}, rt())
    assert part.weight.dtype == torch.float32                     # norm scales are kept in fp32
    x = torch.randn(6, 40, device="cuda")
    ref = P.rmsnorm(x.double().cpu().numpy(), w.to(torch.bfloat16).double().numpy(), 1e-3)
    assert H.rel_to_max(part.forward(x).cpu().numpy(), ref) < 1e-6


def test_position_part_tables():
    from llmi_b200.parts import get_part
    part = get_part("position", "rotary_half")(spec("rotary_half", {"head_dim": 48, "theta": 130000.0}), {}, rt())
    assert part.rotary_dim == 48
    assert np.array_equal(part.inv_freq.cpu().numpy(), P.rope_inv_freq(48, 130000.0))
    none = get_part("position", "none")(spec("none", {}), {}, rt())
    assert none.rotary_dim == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ffn_part(dtype):
    from llmi_b200.parts import get_part
    W, F = 72, 200
    t = {"gate_proj.weight": torch.randn(F, W) * 0.1, "up_proj.weight": torch.randn(F, W) * 0.1,
         "down_proj.weight": torch.randn(W, F) * 0.1}
    t = {k: v.to(dtype) for k, v in t.items()}
    part = get_part("ffn", "swiglu")(spec("swiglu", {"width": W, "inner": F}), t, rt(dtype))
    h = torch.randn(5, W, device="cuda").to(dtype)
    x = torch.randn(5, W, device="cuda")
    before = x.clone()
    part.forward(h, x, None)
    ref = before.double().cpu().numpy() + P.swiglu_ffn(h.double().cpu().numpy(), *(t[k].double().numpy() for k in
                                                       ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
    assert H.rel_to_max(x.cpu().numpy(), ref) < (1e-5 if dtype == torch.float32 else 1e-2)


def test_embedding_and_tied_head():
    from llmi_b200.parts import get_part
    r = rt()
    table = torch.randn(50, 24)
    emb = get_part("embedding", "token_table")(spec("token_table", {"vocab": 50, "width": 24}), {"weight": table}, r)
    head = get_part("head", "linear_head")(spec("linear_head", {"vocab": 50, "width": 24, "tied": True}), {}, r, embedding=emb)
    assert head.weight.data_ptr() == emb.weight.data_ptr() and head.weight_bytes() == 0
    ids = torch.tensor([3, 49, 0], dtype=torch.int32, device="cuda")
    x = emb.forward(ids, None)
    assert torch.equal(x.cpu(), table[[3, 49, 0]])
    logits = head.forward(x.clone())
    assert H.rel_to_max(logits.cpu().numpy(), (table[[3, 49, 0]].double() @ table.double().T).numpy()) < 1e-5


# -- another order of layers ---------------------------------------------------------------------

def test_schedule_is_data(model_dirs):
    """A schedule that runs layer 0 twice (each call with a cache of its own) equals a plain model
    whose layer list is [0, 1, 0]."""
    import dataclasses
    import llmi_b200 as L
    from llmi_b200.config import read_model_config
    from llmi_b200.engine.model import Model
    from llmi_b200.parts import ScheduleEntry
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.weights import SafetensorsFile, load_tensors
    d = model_dirs("A", "F32")
    arch, cfg = read_model_config(d)
    base = arch.model_spec(cfg)
    twice = dataclasses.replace(base, schedule=(ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0)))
    f = SafetensorsFile(d + "/model.safetensors")
    tensors = load_tensors(f, {n: t.shape for n, t in expected_tensors(base).items()}, "cuda:0")
    model = Model(twice, tensors, torch.float32)
    cache = model.new_cache(128)
    assert cache.kv_groups[0].n_calls == 3
    pcfg, pw = P.read_model(d)
    pw3 = dict(pw)
    for k, v in pw.items():
        if k.startswith("model.layers.0."):
            pw3[k.replace("layers.0.", "layers.2.")] = v
    toks = list(range(3, 90, 2))
    ref = P.forward(dict(pcfg, num_hidden_layers=3), pw3, toks)
    s = cache.alloc_slot()
    a = model.step(cache, [L.SequenceStep(s, toks[:30], list(range(30)))]).cpu().numpy().copy()
    b = np.concatenate([model.step(cache, [L.SequenceStep(s, [t], [0])]).cpu().numpy() for t in toks[30:]])
    assert H.rel_to_max(np.concatenate([a, b]), ref) < H.TOL["float32"]


def test_reading_another_calls_cache(model_dirs):
    """A call that reads another call's cache keeps none of its own and writes nothing; prefill and
    token-by-token decoding still agree."""
    import dataclasses
    import llmi_b200 as L
    from llmi_b200.config import read_model_config
    from llmi_b200.engine.model import Model
    from llmi_b200.parts import ScheduleEntry
    from llmi_b200.parts.build import expected_tensors
    from llmi_b200.weights import SafetensorsFile, load_tensors
    d = model_dirs("A", "F32")
    arch, cfg = read_model_config(d)
    base = arch.model_spec(cfg)
    shared = dataclasses.replace(base, schedule=(ScheduleEntry(0), ScheduleEntry(1, cache_of=0)))
    tensors = load_tensors(SafetensorsFile(d + "/model.safetensors"),
                           {n: t.shape for n, t in expected_tensors(base).items()}, "cuda:0")
    model = Model(shared, tensors, torch.float32)
    cache = model.new_cache(128)
    assert cache.kv_groups[0].n_calls == 1 and [b.writes for b in cache.bindings] == [True, False]
    toks = list(range(5, 60))
    s = cache.alloc_slot()
    whole = model.step(cache, [L.SequenceStep(s, toks, list(range(len(toks))))]).cpu().numpy().copy()
    cache.free_slot(s)
    s = cache.alloc_slot()
    a = model.step(cache, [L.SequenceStep(s, toks[:20], list(range(20)))]).cpu().numpy().copy()
    b = np.concatenate([model.step(cache, [L.SequenceStep(s, [t], [0])]).cpu().numpy() for t in toks[20:]])
    assert H.rel_to_max(np.concatenate([a, b]), whole.astype(np.float64)) < 2e-6


# -- a toy mixer with state of its own -----------------------------------------------------------

def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    """An exponential-average mixer: state s ← decay·s + h_t per sequence, output s·Wᵀ.  It is
    defined here, asks the cache for a fixed-size state, and runs through the library's model, step
    function and trace replayer unchanged, prefill and decode, with slots reused."""
    import llmi_b200 as L
    from llmi_b200.cache import StateRequest
    from llmi_b200.config.registry import Architecture
    from llmi_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl
    from llmi_b200.parts.registry import register_part

    class ToyAverage:
        @classmethod
        def declare(cls, spec):
            w = spec.params["width"]
            return {"mix.weight": TensorDecl((w, w))}

        def __init__(self, spec, tensors, rt, **_):
            self.rt, self.width, self.decay = rt, spec.params["width"], spec.params["decay"]
            self.w = rt.to_f32(tensors["mix.weight"])

        def cache_request(self):
            return StateRequest((self.width,), torch.float32)

        def forward(self, h, x, ctx, binding):
            state = binding.group.data[binding.index]                 # [slots, width]
            starts = ctx.seq_q_start.cpu().tolist()
            slots = ctx.seq_slot.cpu().tolist()
            for i, slot in enumerate(slots):
                if slot < 0:
                    continue
                for t in range(starts[i], starts[i + 1]):
                    state[slot] = self.decay * state[slot] + h[t].float()
                    x[t] += state[slot] @ self.w.T

    register_part("mixer", "toy_average", ToyAverage, replace=True)

    def toy_spec(c):
        w = c["width"]
        layers = tuple(LayerSpec("prenorm", PartSpec("rms", {"width": w, "eps": 1e-5}, f"l{i}.n1."),
                                 PartSpec("toy_average", {"width": w, "decay": c["decay"]}, f"l{i}."),
                                 PartSpec("rms", {"width": w, "eps": 1e-5}, f"l{i}.n2."),
                                 PartSpec("swiglu", {"width": w, "inner": 2 * w}, f"l{i}.ffn.")) for i in range(c["layers"]))
        return ModelSpec("ToyAverageLM", c["vocab"], w, 4096, PartSpec("token_table", {"vocab": c["vocab"], "width": w}, "emb."),
                         layers, tuple(ScheduleEntry(i) for i in range(c["layers"])),
                         PartSpec("rms", {"width": w, "eps": 1e-5}, "final."),
                         PartSpec("linear_head", {"vocab": c["vocab"], "width": w, "tied": True}, "head."))

    L.register_architecture(Architecture("ToyAverageLM", lambda root: dict(root), toy_spec), replace=True)
    cfg = {"architectures": ["ToyAverageLM"], "width": 40, "layers": 2, "vocab": 90, "decay": 0.5}
    L.write_random_model(str(tmp_path), cfg, 7)
    model = L.load(str(tmp_path), "float32")
    cache = model.new_cache(256)
    assert not cache.kv_groups and cache.state_groups[0].data.shape == (2, 4, 40)

    reqs = {"a": list(range(1, 30)), "b": list(range(40, 47)), "c": list(range(60, 85))}
    s1, m1 = H.trace_whole(reqs)
    s2, m2 = H.trace_batches(reqs, 2, {"a": 5, "b": 7, "c": 1})
    whole = H.collect(s1, H.replay(model, s1, 256, poison=False), 90)
    cut = H.collect(s2, H.replay(model, s2, 256, poison=False), 90)
    for r in reqs:
        assert np.isfinite(whole[r]).all()
        assert H.rel_to_max(cut[r], whole[r].astype(np.float64)) < 1e-5
    # the state really is per sequence: a different history gives different logits at the same token
    s3, _ = H.trace_whole({"a": [9] + reqs["a"][1:]})
    other = H.collect(s3, H.replay(model, s3, 256, poison=False), 90)
    assert H.rel_to_max(other["a"][1:2], whole["a"][1:2].astype(np.float64)) > 1e-4


# -- layers with different cache needs -----------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_and_global_layers_keep_separate_cache_groups(tmp_path, dtype):
    """A toy architecture whose first layer sees all keys and whose second sees a window of 40: the two
    get cache groups (page pools) of their own, the windowed one gives pages back while decoding, and
    prefill, decode and batches agree with the plain formulas."""
    import llmi_b200 as L
    from llmi_b200.config.registry import Architecture
    from llmi_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    W, NH, NKV, HD, F, V, WIN = 128, 4, 2, 64, 192, 300, 40

    def toy_spec(c):
        def layer(i, window):
            p = f"blk{i}."
            pos = PartSpec("rotary_half", {"head_dim": HD, "theta": 10000.0})
            return LayerSpec("prenorm", PartSpec("rms", {"width": W, "eps": 1e-5}, p + "n1."),
                             PartSpec("gqa", {"width": W, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD, "bias": False,
                                              "window": window, "position": pos}, p + "attn."),
                             PartSpec("rms", {"width": W, "eps": 1e-5}, p + "n2."),
                             PartSpec("swiglu", {"width": W, "inner": F}, p + "ffn."))
        return ModelSpec("ToyWindowLM", V, W, 2048, PartSpec("token_table", {"vocab": V, "width": W}, "emb."),
                         (layer(0, 0), layer(1, WIN)), (ScheduleEntry(0), ScheduleEntry(1)),
                         PartSpec("rms", {"width": W, "eps": 1e-5}, "final."),
                         PartSpec("linear_head", {"vocab": V, "width": W, "tied": True}, "head."))

    L.register_architecture(Architecture("ToyWindowLM", lambda root: dict(root), toy_spec), replace=True)
    storage = torch.float32 if dtype == "float32" else torch.bfloat16
    L.write_random_model(str(tmp_path), {"architectures": ["ToyWindowLM"]}, 3, storage)
    model = L.load(str(tmp_path), dtype)
    cache = model.new_cache(64 * 12)
    assert len(cache.kv_groups) == 2 and sorted(g.request.window for g in cache.kv_groups) == [0, WIN]

    w = P.read_safetensors(str(tmp_path / "model.safetensors"))

    def plain(tokens):
        T = len(tokens)
        x = P.embedding(w["emb.weight"], tokens)
        inv = P.rope_inv_freq(HD, 10000.0)
        for i, window in ((0, 0), (1, WIN)):
            p = f"blk{i}."
            h = P.rmsnorm(x, w[p + "n1.weight"], 1e-5)
            q = P.linear(h, w[p + "attn.q_proj.weight"]).reshape(T, NH, HD)
            k = P.linear(h, w[p + "attn.k_proj.weight"]).reshape(T, NKV, HD)
            v = P.linear(h, w[p + "attn.v_proj.weight"]).reshape(T, NKV, HD)
            pos = np.arange(T)
            a = P.attention(P.rope(q, pos, inv), P.rope(k, pos, inv), v, window).reshape(T, NH * HD)
            x = x + P.linear(a, w[p + "attn.o_proj.weight"])
            h = P.rmsnorm(x, w[p + "n2.weight"], 1e-5)
            x = x + P.swiglu_ffn(h, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
        return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["emb.weight"])

    rng = np.random.default_rng(4)
    reqs = {"a": rng.integers(0, V, 150).tolist(), "b": rng.integers(0, V, 47).tolist(), "c": rng.integers(0, V, 260).tolist()}
    refs = {r: plain(t) for r, t in reqs.items()}
    tol = H.TOL[dtype]
    for steps, most in (H.trace_whole(reqs), H.trace_last_decoded(reqs, 100), H.trace_batches(reqs, 3, {"a": 30, "b": 47, "c": 129})):
        got = H.collect(steps, H.replay(model, steps, max(most, 64 * 12)), V)
        for r in reqs:
            assert np.isfinite(got[r]).all()
            assert H.rel_to_max(got[r], refs[r]) < tol, r
    # long decoding keeps the windowed group's pages bounded: after 260 positions it holds at most 2 pages
    s = cache.alloc_slot()
    model.step(cache, [L.SequenceStep(s, reqs["c"][:200], [])])
    for t in reqs["c"][200:]:
        model.step(cache, [L.SequenceStep(s, [t], [])])
    win_group = [g for g in cache.kv_groups if g.request.window][0]
    all_group = [g for g in cache.kv_groups if not g.request.window][0]
    assert sum(p >= 0 for p in win_group.pool.table(s)) <= 2 and sum(p >= 0 for p in all_group.pool.table(s)) == 5
    cache.free_slot(s)
    cache.check()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,bias", [(4, 2, 64, False), (5, 1, 24, True), (6, 6, 32, False)])
def test_attention_mixer_part_alone(dtype, nh, nkv, hd, bias):
    """The grouped-query attention part by itself, on a cache of its own: a prompt in one step, then a few
    single tokens, against the plain attention block (projections, rotation, attention, output projection)."""
    from llmi_b200.cache import SequenceCache
    from llmi_b200.cache.storage import CacheBinding
    from llmi_b200.engine.batch import SequenceStep, StepBuffers, plan_step
    from llmi_b200.parts import get_part
    W = 136
    r = rt(dtype)
    names = {"q_proj.weight": (nh * hd, W), "k_proj.weight": (nkv * hd, W), "v_proj.weight": (nkv * hd, W),
             "o_proj.weight": (W, nh * hd)}
    if bias:
        names.update({"q_proj.bias": (nh * hd,), "k_proj.bias": (nkv * hd,), "v_proj.bias": (nkv * hd,)})
    t = {n: (torch.randn(*s) * 0.08).to(dtype) for n, s in names.items()}
    pos = spec("rotary_half", {"head_dim": hd, "theta": 5000.0})
    part = get_part("mixer", "gqa")(spec("gqa", {"width": W, "n_heads": nh, "n_kv_heads": nkv, "head_dim": hd, "bias": bias,
                                                 "window": 0, "position": pos}), t, r)
    req = part.cache_request()
    cache = SequenceCache([(req, 1)], [], 256, 4096, dtype, "cuda:0")
    binding = CacheBinding(cache.kv_groups[0], 0)
    buffers = StepBuffers(torch.device("cuda:0"))
    T, extra = 70, 5
    h_all = (torch.randn(T + extra, W) * 0.5).to(dtype)
    slot = cache.alloc_slot()
    outs = []
    for lo, hi in [(0, T)] + [(T + i, T + i + 1) for i in range(extra)]:
        ctx = plan_step(cache, [SequenceStep(slot, [0] * (hi - lo), [])], 10, buffers)
        x = torch.zeros(hi - lo, W, device="cuda")
        part.forward(h_all[lo:hi].cuda().contiguous(), x, ctx, binding)
        outs.append(x.cpu())
    got = torch.cat(outs).double().numpy()
    # the plain block without its norm: q/k/v projections (+bias), rotation, attention, output projection
    w64 = {k: v.double().numpy() for k, v in t.items()}
    hh = h_all.double().numpy()
    n = T + extra
    q = P.linear(hh, w64["q_proj.weight"], w64.get("q_proj.bias")).reshape(n, nh, hd)
    k = P.linear(hh, w64["k_proj.weight"], w64.get("k_proj.bias")).reshape(n, nkv, hd)
    v = P.linear(hh, w64["v_proj.weight"], w64.get("v_proj.bias")).reshape(n, nkv, hd)
    inv = P.rope_inv_freq(hd, 5000.0)
    a = P.attention(P.rope(q, np.arange(n), inv), P.rope(k, np.arange(n), inv), v).reshape(n, nh * hd)
    ref = P.linear(a, w64["o_proj.weight"])
    assert H.rel_to_max(got, ref) < (2e-5 if dtype == torch.float32 else 1.5e-2)


# -- a feed-forward with routing and another position encoding, both defined here ------------------

def test_toy_routed_ffn_and_learned_positions(tmp_path):
    """Two more toy parts registered from outside the library: a feed-forward that routes every token to
    the best of three experts (router logits in 32-bit) and a position encoding that is a learned table
    added after the embedding lookup (held by the embedding part, with a tensor of its own; keys are
    stored unrotated).  The library's model, cache, step and replay run them unchanged; whole prompts,
    token-by-token decoding and unequal batches agree with the plain formulas."""
    import llmi_b200 as L
    from llmi_b200.config.registry import Architecture
    from llmi_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorDecl
    from llmi_b200.parts.position import PositionEncoding
    from llmi_b200.parts.registry import register_part

    W, NH, NKV, HD, F, V, E, MAXPOS = 64, 4, 2, 16, 48, 120, 3, 256

    class LearnedPositions(PositionEncoding):
        @classmethod
        def declare(cls, spec):
            return {"table": TensorDecl((spec.params["max_pos"], spec.params["width"]), "table")}

        def __init__(self, spec, tensors, rt, **_):
            self.table = rt.to_f32(tensors["table"])

        def at_embedding(self, x, ctx):
            live = ctx.tok_seq >= 0                                   # padding tokens stay zero
            x[live] += self.table[ctx.tok_pos[live].long()]

    class Top1Experts:
        @classmethod
        def declare(cls, spec):
            w, f, e = spec.params["width"], spec.params["inner"], spec.params["experts"]
            d = {"router.weight": TensorDecl((e, w))}
            for i in range(e):
                d[f"experts.{i}.up.weight"] = TensorDecl((f, w))
                d[f"experts.{i}.down.weight"] = TensorDecl((w, f))
            return d

        def __init__(self, spec, tensors, rt, **_):
            self.e = spec.params["experts"]
            self.router = rt.to_f32(tensors["router.weight"])
            self.up = [rt.to_f32(tensors[f"experts.{i}.up.weight"]) for i in range(self.e)]
            self.down = [rt.to_f32(tensors[f"experts.{i}.down.weight"]) for i in range(self.e)]

        def forward(self, h, x, ctx):
            h = h.float()
            choice = (h @ self.router.T).argmax(dim=1)                 # router logits in 32-bit
            for i in range(self.e):                                    # experts in a fixed order
                rows = (choice == i).nonzero().flatten()
                if rows.numel():
                    x[rows] += torch.relu(h[rows] @ self.up[i].T) @ self.down[i].T

    register_part("position", "toy_learned", LearnedPositions, replace=True)
    register_part("ffn", "toy_top1", Top1Experts, replace=True)

    def toy_spec(c):
        layers = tuple(LayerSpec("prenorm", PartSpec("rms", {"width": W, "eps": 1e-5}, f"l{i}.n1."),
                                 PartSpec("gqa", {"width": W, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD, "bias": False,
                                                  "position": PartSpec("none", {})}, f"l{i}.attn."),
                                 PartSpec("rms", {"width": W, "eps": 1e-5}, f"l{i}.n2."),
                                 PartSpec("toy_top1", {"width": W, "inner": F, "experts": E}, f"l{i}.moe.")) for i in range(2))
        emb = PartSpec("token_table", {"vocab": V, "width": W,
                                       "position": PartSpec("toy_learned", {"max_pos": MAXPOS, "width": W}, "pos.")}, "emb.")
        return ModelSpec("ToyRoutedLM", V, W, MAXPOS, emb, layers, (ScheduleEntry(0), ScheduleEntry(1)),
                         PartSpec("rms", {"width": W, "eps": 1e-5}, "final."),
                         PartSpec("linear_head", {"vocab": V, "width": W, "tied": False}, "head."))

    L.register_architecture(Architecture("ToyRoutedLM", lambda root: dict(root), toy_spec), replace=True)
    L.write_random_model(str(tmp_path), {"architectures": ["ToyRoutedLM"]}, 11, torch.float32)
    model = L.load(str(tmp_path), "float32")
    w = P.read_safetensors(str(tmp_path / "model.safetensors"))
    assert w["emb.pos.table"].shape == (MAXPOS, W) and w["l1.moe.experts.2.down.weight"].shape == (W, F)

    used = set()

    def plain(tokens):
        T = len(tokens)
        x = P.embedding(w["emb.weight"], tokens) + w["emb.pos.table"][:T].astype(np.float64)
        for i in range(2):
            p = f"l{i}."
            h = P.rmsnorm(x, w[p + "n1.weight"], 1e-5)
            q = P.linear(h, w[p + "attn.q_proj.weight"]).reshape(T, NH, HD)
            k = P.linear(h, w[p + "attn.k_proj.weight"]).reshape(T, NKV, HD)
            v = P.linear(h, w[p + "attn.v_proj.weight"]).reshape(T, NKV, HD)
            x = x + P.linear(P.attention(q, k, v, 0).reshape(T, NH * HD), w[p + "attn.o_proj.weight"])
            h = P.rmsnorm(x, w[p + "n2.weight"], 1e-5)
            choice = P.linear(h, w[p + "moe.router.weight"]).argmax(axis=1)
            for t in range(T):
                e = int(choice[t])
                used.add((i, e))
                up = np.maximum(P.linear(h[t:t + 1], w[p + f"moe.experts.{e}.up.weight"]), 0)
                x[t] = x[t] + P.linear(up, w[p + f"moe.experts.{e}.down.weight"])[0]
        return P.linear(P.rmsnorm(x, w["final.weight"], 1e-5), w["head.weight"])

    rng = np.random.default_rng(5)
    reqs = {"a": rng.integers(0, V, 90).tolist(), "b": rng.integers(0, V, 33).tolist(), "c": rng.integers(0, V, 140).tolist()}
    refs = {r: plain(t) for r, t in reqs.items()}
    assert len(used) == 2 * E                                           # every expert of every layer saw tokens
    for steps, most in (H.trace_whole(reqs), H.trace_last_decoded(reqs, 32), H.trace_batches(reqs, 2, {"a": 30, "b": 33, "c": 70})):
        got = H.collect(steps, H.replay(model, steps, max(most, 512)), V)
        for r in reqs:
            assert np.isfinite(got[r]).all()
            assert H.rel_to_max(got[r], refs[r]) < 2e-5, r


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_arrangement_with_other_slots_without_touching_the_library(tmp_path, dtype):
    """A layer is an arrangement and the parts in its named slots.  Here an arrangement defined in the test puts a norm
    AFTER the mixer as well ("sandwich": x += post_norm(attention(norm(x)))), one layer has a feed-forward and the
    other has none, and the library's own norm, attention and feed-forward parts fill the slots: spec, builder,
    weights, cache, step and replay are the library's, unchanged."""
    import llmi_b200 as L
    from llmi_b200.config.registry import Architecture
    from llmi_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from llmi_b200.parts.registry import register_part

    W, NH, NKV, HD, F, V, MAXPOS, EPS, THETA = 80, 5, 1, 16, 112, 150, 256, 1e-5, 20000.0

    class Sandwich:
        """x += post_mixer_norm(mixer(mixer_norm(x))); then, if the layer has them, x += ffn(ffn_norm(x))."""

        def __init__(self, mixer_norm, mixer, post_mixer_norm, ffn_norm=None, ffn=None):
            self.mixer_norm, self.mixer, self.post, self.ffn_norm, self.ffn = mixer_norm, mixer, post_mixer_norm, ffn_norm, ffn

        def forward(self, x, ctx, binding):
            branch = torch.zeros_like(x)                         # the library's mixers ADD their output to what they are given
            self.mixer.forward(self.mixer_norm.forward(x), branch, ctx, binding)
            x += self.post.forward(branch, scratch_name="sandwich_post").float()
            if self.ffn is not None:
                self.ffn.forward(self.ffn_norm.forward(x), x, ctx)

    register_part("block", "toy_sandwich", Sandwich, replace=True)

    def norm(prefix):
        return PartSpec("rms", {"width": W, "eps": EPS}, prefix)

    def toy_spec(c):
        pos = PartSpec("rotary_half", {"head_dim": HD, "theta": THETA})
        layers = []
        for i in range(2):
            p = f"model.layers.{i}."
            layers.append(LayerSpec(
                "toy_sandwich", mixer_norm=norm(p + "input_layernorm."),
                mixer=PartSpec("gqa", {"width": W, "n_heads": NH, "n_kv_heads": NKV, "head_dim": HD, "bias": False,
                                       "position": pos}, p + "self_attn."),
                ffn_norm=norm(p + "post_attention_layernorm.") if i == 0 else None,
                ffn=PartSpec("swiglu", {"width": W, "inner": F}, p + "mlp.") if i == 0 else None,
                more=(("post_mixer_norm", "norm", norm(p + "post_mixer_norm.")),)))
        return ModelSpec("ToySandwichLM", V, W, MAXPOS, PartSpec("token_table", {"vocab": V, "width": W}, "model.embed_tokens."),
                         tuple(layers), (ScheduleEntry(0), ScheduleEntry(1)), norm("model.norm."),
                         PartSpec("linear_head", {"vocab": V, "width": W, "tied": True}, "lm_head."))

    L.register_architecture(Architecture("ToySandwichLM", lambda root: dict(root), toy_spec), replace=True)
    L.write_random_model(str(tmp_path), {"architectures": ["ToySandwichLM"]}, 3, torch.float32 if dtype == "float32" else torch.bfloat16)
    model = L.load(str(tmp_path), dtype)
    w = P.read_safetensors(str(tmp_path / "model.safetensors"))
    assert "model.layers.1.mlp.up_proj.weight" not in w and "model.layers.1.post_mixer_norm.weight" in w
    assert model.weight_bytes() > 0
    sz = dict(nh=NH, nkv=NKV, hd=HD, eps=EPS, bias=False)

    def plain(tokens):
        T = len(tokens)
        inv = P.rope_inv_freq(HD, THETA)
        x = P.embedding(w["model.embed_tokens.weight"], tokens)
        for i in range(2):
            p = f"model.layers.{i}."
            x = x + P.rmsnorm(P.attention_block(x, w, p, sz, np.arange(T), inv), w[p + "post_mixer_norm.weight"], EPS)
            if i == 0:
                h = P.rmsnorm(x, w[p + "post_attention_layernorm.weight"], EPS)
                x = x + P.swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
        return P.linear(P.rmsnorm(x, w["model.norm.weight"], EPS), w["model.embed_tokens.weight"])

    rng = np.random.default_rng(6)
    reqs = {"a": rng.integers(0, V, 70).tolist(), "b": rng.integers(0, V, 9).tolist(), "c": rng.integers(0, V, 130).tolist()}
    refs = {r: plain(t) for r, t in reqs.items()}
    for steps, most in (H.trace_whole(reqs), H.trace_last_decoded(reqs, 32), H.trace_batches(reqs, 3, {"a": 30, "b": 9, "c": 70}),
                        H.trace_portions(reqs, 50)):
        got = H.collect(steps, H.replay(model, steps, max(most, 512)), V)
        for r in reqs:
            assert np.isfinite(got[r]).all()
            assert H.rel_to_max(got[r], refs[r]) < H.TOL[dtype], r
