"""Decode and prefill throughput of the library at SmolLM2-1.7B shape (random bf16 weights, one B200).

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload smollm2-360m|smollm2-135m [--workload-dtypes bfloat16,float32]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 and context 4096 (a
"step" is one decode step of the whole batch), timed on the device with CUDA events around
exactly K steps after W warm-up steps.  ``e2e`` is the same through the public entry point
(``Model.step_and_choose``): host token ids in, host token ids out, every step.  ``prefill`` is
one 2,048-token prompt; ``points`` are decode at batch 1 and 64; ``roofline`` relates the decode
step to HBM bandwidth: (every weight once + the cache of the live requests) / step time.
Peaks come from MEASURED_PEAKS.json beside this file when present, else from the fallback
figures (6.65 TB/s copy, 1.59 PFLOP/s bf16).  Token ids are seeded uniform random numbers and
the cache of the decode runs is filled with random keys and values instead of a real prefill
(the time of a step does not depend on their values).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# SmolLM2-1.7B layer sizes (BASELINE.json configs[2])
CONFIG = {
    "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 32,
    "num_key_value_heads": 32, "head_dim": 64, "intermediate_size": 8192, "vocab_size": 49152, "rope_theta": 130000.0,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu",
}
FULL_LAYERS = 24
CONTEXT = 4096
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None
        self.begin = self.end = None

    def start(self):
        """Start sampling (the tool takes a moment to come up: call this before the warm-up)."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark_begin(self):
        self.begin = len(self.rows)

    def mark_end(self):
        self.end = len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        rows = self.rows[self.begin:self.end] if self.begin is not None and self.end is not None else self.rows
        where = "timed region"
        if not rows:                      # a region shorter than one sampling period: the samples around it
            rows, where = self.rows[max(0, (self.begin or 0) - 2):(self.end or 0) + 2], "around the timed region"
        sm = sorted(int(r[0]) for r in rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "sampled": where}


def fill_cache(cache, model, batch, start_len):
    """Slots whose caches hold ``start_len`` positions of random keys and values."""
    import torch
    for g in cache.kv_groups:
        g.k.normal_(0, 0.5)
        g.v.normal_(0, 0.5)
    slots = []
    for _ in range(batch):
        s = cache.alloc_slot()
        cache.extend(s, start_len)
        slots.append(s)
    torch.cuda.synchronize()
    return slots


def decode_run(model, batch, context, steps, warmup, e2e=False, clocks=None):
    """Decode `steps` steps ending at `context`; returns (ms per step, launches, h2d, d2h bytes per step)."""
    import torch
    from llmi_b200 import SamplingParams, SequenceStep
    from llmi_b200.engine.graphs import DecodeGraphs
    from llmi_b200.ops import kernels
    from llmi_b200.sampling import Sampler
    total = warmup + steps
    start = context - total
    cache = model.new_cache(batch * ((context + 63) // 64) * 64, n_slots=batch)
    slots = fill_cache(cache, model, batch, start)
    sampler = Sampler(SamplingParams(), model.rt)
    if model._graphs is None:
        model._graphs = DecodeGraphs(model)
    rng = torch.Generator().manual_seed(batch)
    toks = torch.randint(0, model.vocab_size, (batch,), generator=rng).tolist()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = h2d = d2h = 0
    for i in range(total):
        if i == warmup:
            torch.cuda.synchronize()
            if clocks:
                clocks.mark_begin()
            launches0 = kernels.launch_count()
            e0.record()
        seqs = [SequenceStep(s, [t], [0]) for s, t in zip(slots, toks)]
        if e2e:
            ids = model.step_and_choose(cache, seqs, sampler)          # host ids in, host ids out
            toks = ids.tolist()
            if i >= warmup:
                h2d += model.last_h2d_bytes
                d2h += ids.numel() * 4
        else:
            model._graphs.step(cache, seqs, sampler)
    e1.record()
    torch.cuda.synchronize()
    if clocks:
        clocks.mark_end()
    ms = e0.elapsed_time(e1) / steps
    launches = kernels.launch_count() - launches0
    kernels.check_device_errors(model.device)
    cache_bytes = batch * (context - steps / 2.0) * cache.bytes_per_token()
    for s in slots:
        cache.free_slot(s)
    del cache
    torch.cuda.empty_cache()
    return ms, launches, h2d / max(steps, 1), d2h / max(steps, 1), cache_bytes


def prefill_run(model, tokens, iters=5):
    import torch
    from llmi_b200 import SequenceStep
    cache = model.new_cache(((tokens + 63) // 64) * 64)
    ids = torch.randint(0, model.vocab_size, (tokens,), generator=torch.Generator().manual_seed(1)).tolist()
    times = []
    for i in range(iters + 2):
        s = cache.alloc_slot()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        model.step(cache, [SequenceStep(s, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        cache.free_slot(s)
        if i >= 2:
            times.append(e0.elapsed_time(e1))
    return sorted(times)[len(times) // 2]


def prefill_flops(cfg, layers, T):
    H, nh, nkv, hd, F, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                            cfg["intermediate_size"], cfg["vocab_size"])
    per_token = layers * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * F)
    attn = layers * 4 * nh * hd * (T * (T + 1) // 2)          # QK^T and PV over the causal half
    return 2 * T * per_token + attn + 2 * H * V              # the head runs on the last row only


# The other two shapes of the benchmark set: whole requests through generate() (prefill and decoding in one time)
WORKLOADS = {
    "smollm2-360m": {
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 32, "hidden_size": 960, "num_attention_heads": 15,
                   "num_key_value_heads": 5, "head_dim": 64, "intermediate_size": 2560, "vocab_size": 49152, "rope_theta": 100000.0,
                   "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"},
        "prompts": lambda rng: [int(n) for n in rng.integers(16, 1025, 8)], "max_new": 256, "max_new_fp32": 256,
        "what": "8 prompts of 16..1,024 uniform random ids, 256 new tokens each"},
    "smollm2-135m": {
        "config": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 30, "hidden_size": 576, "num_attention_heads": 9,
                   "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1536, "vocab_size": 49152, "rope_theta": 100000.0,
                   "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192, "hidden_act": "silu"},
        "prompts": lambda rng: [512] * 64, "max_new": 512, "max_new_fp32": 64,
        "what": "64 prompts of 512 uniform random ids, 512 new tokens each (64 in fp32)"},
}


def workload_run(name, dtypes):
    """One of the other benchmark shapes through the public entry point; prints one JSON line."""
    import numpy as np
    import torch
    import llmi_b200 as L
    wl = WORKLOADS[name]
    rng = np.random.default_rng(0)
    lens = wl["prompts"](rng)
    V = wl["config"]["vocab_size"]
    prompts = [rng.integers(0, V, n).tolist() for n in lens]
    out = {"workload": name, "what": wl["what"], "impl": "ours", "data": "synthetic (random weights, uniform random token ids)",
           "prompt_tokens": int(sum(lens)), "runs": {}}
    for dtype in dtypes:
        max_new = wl["max_new"] if dtype == "bfloat16" else wl["max_new_fp32"]
        model = L.random_model(wl["config"], seed=0, dtype=dtype, on_device=True)
        L.generate(model, prompts[:2], max_new=4, ignore_eos=True)          # builds the kernels' one-time state
        best = None
        for _ in range(2):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            got, info = L.generate(model, prompts, max_new=max_new, ignore_eos=True, return_details=True)
            torch.cuda.synchronize()
            sec = time.perf_counter() - t0
            best = sec if best is None else min(best, sec)
        new = sum(len(g) for g in got)
        out["runs"][dtype] = {"seconds": round(best, 4), "new_tokens": new, "new_tokens_per_s": round(new / best, 1),
                              "steps": info["steps"], "batches": info["batches"]}
        del model
        torch.cuda.empty_cache()
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the full model (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --only prefill: another prompt length")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print its numbers (for profiling one kernel class; not a bench line)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=None,
                    help="run one of the other benchmark shapes whole, through generate(), and print its own JSON line")
    ap.add_argument("--workload-dtypes", default="bfloat16", help="comma-separated: bfloat16, float32")
    ap.add_argument("--kv-heads", type=int, default=None,
                    help="with --only: another number of key/value heads (grouped queries), to profile their kernels")
    args = ap.parse_args()

    if args.impl == "reference":
        if args.gpus != 1:
            print(json.dumps({"impl": "reference", "unavailable": "the reference runs on the CPU of one machine; --gpus must be 1"}))
            return 0
        # the unmodified reference through its own command line (a CMake C++ project: the offline pip install has
        # nothing to install — 'Neither setup.py nor pyproject.toml found' — so it is built with its own CMake files)
        from baseline import reference_arm
        return reference_arm.main(dict(CONFIG, num_hidden_layers=args.layers), args.batch, args.context, PREFILL_TOKENS,
                                  args.steps, args.warmup, FULL_LAYERS)
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    if args.workload:
        return workload_run(args.workload, [d.strip() for d in args.workload_dtypes.split(",") if d.strip()])
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    import torch
    import llmi_b200 as L
    pk, pk_kind = peaks()
    cfg = dict(CONFIG, num_hidden_layers=args.layers)
    if args.kv_heads is not None:
        if args.only is None:
            print("bench.py: --kv-heads changes the model's shape; it goes with --only (no bench line)")
            return 2
        cfg["num_key_value_heads"] = args.kv_heads
    t0 = time.time()
    model = L.random_model(cfg, seed=0, dtype="bfloat16", on_device=True)
    weight_bytes = model.weight_bytes()

    if args.only == "prefill":
        T = args.prefill_tokens
        pre_ms = prefill_run(model, T, iters=3)
        frac = prefill_flops(cfg, args.layers, T) / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)
        print(json.dumps({"only": "prefill", "ms": round(pre_ms, 3), "tokens": T, "layers": args.layers,
                          "tokens_per_s": round(T * 1000.0 / pre_ms, 1), "frac_of_bf16_peak": round(frac, 4), "peaks": pk_kind}))
        return 0
    if args.only == "decode":
        ms, launches, _, _, cache_bytes = decode_run(model, args.batch, args.context, steps, warmup)
        gbs = (weight_bytes + cache_bytes) / (ms * 1e-3) / 1e9
        print(json.dumps({"only": "decode", "ms_per_step": round(ms, 4), "batch": args.batch, "context": args.context,
                          "layers": args.layers, "kv_heads": cfg["num_key_value_heads"], "gpu_launches": launches,
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1), "gb_per_s": round(gbs, 1),
                          "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 4), "peaks": pk_kind}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    ms, launches, _, _, cache_bytes = decode_run(model, args.batch, args.context, steps, warmup, clocks=clocks)
    clock_info = clocks.stop()
    value = args.batch * 1000.0 / ms
    ms_e2e, _, h2d, d2h, _ = decode_run(model, args.batch, args.context, steps, warmup, e2e=True)
    step_bytes = weight_bytes + cache_bytes
    achieved = step_bytes / (ms * 1e-3) / 1e9

    pre_ms = prefill_run(model, PREFILL_TOKENS)
    pre_flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, *_ = decode_run(model, b, args.context, min(steps, 32), warmup)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)

    out = {
        "metric": "decode tok/s at batch 8, context 4096 (SmolLM2-1.7B shape)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random weights, uniform random token ids, random cache contents)",
        "impl": "ours",
        "config": {"model": "SmolLM2-1.7B shape", "layers": args.layers, "layers_full": FULL_LAYERS, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied": True, "global_batch": args.batch, "seq_len": args.context,
                   "prefill_tokens": PREFILL_TOKENS, "parallelism": "1 GPU", "weights": "random bf16",
                   "l2": "inputs larger than L2 (a step reads %.1f GB)" % (step_bytes / 1e9), "peaks": pk_kind},
        "e2e": {"value": round(args.batch * 1000.0 / ms_e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
                    "frac": round(pre_flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clock_info,
        "setup_seconds": round(time.time() - t0, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
