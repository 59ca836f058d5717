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
