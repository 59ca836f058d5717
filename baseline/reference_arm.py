"""The reference arm of ``bench.py``: the unmodified reference engine, through its own command line.

The reference (fernandojcardenas/llm-inference-cpp) is a CMake C++ project that runs on the CPU in fp32; its
public entry point for generation is ``llmi-generate`` (apps/llmi-generate/main.cpp:205-264).  This arm

* builds ``llmi-generate`` from an unmodified copy of the reference's sources under ``baseline/_ref/src``
  (``cmake -DLLMI_BUILD_TESTS=OFF -DCMAKE_BUILD_TYPE=Release``; nothing is fetched with the tests off) into
  ``baseline/_ref/build``, unless a binary that runs is there already;
* writes a model folder of the benchmark's layer sizes with this library's seeded random-weights writer
  (bf16 storage; the reference widens every weight to fp32 at load, src/model/model.cpp:185-187);
* runs ``llmi-generate DIR --ids <ids> --max-new N --ignore-eos --json --kv-cache`` — the stock cached greedy
  path, src/model/transformer.cpp:308-327 — and reads ``generate_seconds`` (main.cpp:339-344).

None of this library's models, kernels or engine is on the timed path.  Decode: two runs over the same prompt
that end ``warmup`` and ``warmup + steps`` tokens later; their difference is the time of ``steps`` decode steps
at the benchmark's context.  The reference serves one sequence at a time (src/server/server.cpp:44-50), so a
batch of 8 is eight sequences one after another and its tokens per second are those of one sequence.  Prefill:
one run over 2,048 ids with ``--max-new 1``.  There is no device boundary: ``e2e`` equals ``value``.

Every run loads the model and prefills its whole prompt on the CPU first (minutes at this size), so after the
prefill run the arm estimates what the two decode runs will cost and, if that exceeds what is left of its time
limit (``LLMI_REFERENCE_LIMIT_S``, default 1600 seconds), gives up with an ``unavailable`` line that carries what it
has measured.
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")
# the copy under baseline/_ref/src, else a checkout named by LLMI_REFERENCE_SRC
SRC_CANDIDATES = tuple(c for c in (os.path.join(REF_DIR, "src"), os.environ.get("LLMI_REFERENCE_SRC")) if c)


class Unavailable(Exception):
    def __init__(self, why: str, partial: dict | None = None):
        super().__init__(why)
        self.why, self.partial = why, partial or {}


def _say(msg: str) -> None:
    print(f"[reference arm] {msg}", file=sys.stderr, flush=True)


def find_sources() -> str:
    for src in SRC_CANDIDATES:
        if os.path.exists(os.path.join(src, "CMakeLists.txt")) and os.path.exists(os.path.join(src, "apps", "llmi-generate")):
            return src
    raise Unavailable("the reference's sources are neither under baseline/_ref/src nor where LLMI_REFERENCE_SRC points")


def _runs(binary: str) -> bool:
    """Whether the binary starts on this machine: without arguments it prints its usage and exits with 2."""
    try:
        r = subprocess.run([binary], capture_output=True, text=True, timeout=30)
    except (OSError, subprocess.TimeoutExpired):
        return False
    return r.returncode == 2


def ensure_binary() -> str:
    """``llmi-generate`` built from the unmodified sources; built now if none that runs is there."""
    for build in (os.path.join(REF_DIR, "build"), os.path.join(REF_DIR, "build-local")):
        binary = os.path.join(build, "llmi-generate")
        if os.path.exists(binary) and _runs(binary):
            return binary
    src = find_sources()
    cmake = shutil.which("cmake")
    if cmake is None or shutil.which("g++") is None and shutil.which("c++") is None:
        raise Unavailable("no cmake or no C++ compiler on this machine to build the reference with")
    build = os.path.join(REF_DIR, "build-local" if os.path.exists(os.path.join(REF_DIR, "build")) else "build")
    os.makedirs(build, exist_ok=True)
    gen = ["-G", "Ninja"] if shutil.which("ninja") else []
    _say(f"building llmi-generate from {src} into {build}")
    t0 = time.time()
    for cmd in ([cmake, "-S", src, "-B", build, *gen, "-DCMAKE_BUILD_TYPE=Release", "-DLLMI_BUILD_TESTS=OFF"],
                [cmake, "--build", build, "--target", "llmi-generate", "--parallel", str(os.cpu_count() or 4)]):
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
        if r.returncode != 0:
            raise Unavailable("building the reference failed: " + (r.stderr or r.stdout).strip().splitlines()[-1][:200])
    binary = os.path.join(build, "llmi-generate")
    if not _runs(binary):
        raise Unavailable("the reference's llmi-generate was built but does not start on this machine")
    _say(f"built in {time.time() - t0:.0f} s")
    return binary


def write_model(config: dict, seed: int = 0) -> str:
    """A model folder for the reference to load (reused while it is there and complete)."""
    import torch
    sys.path.insert(0, ROOT)
    from llmi_b200 import write_random_model
    name = "llmi_reference_model_L%d_H%d_V%d_s%d" % (config["num_hidden_layers"], config["hidden_size"],
                                                    config["vocab_size"], seed)
    d = os.path.join(tempfile.gettempdir(), name)
    done = os.path.join(d, ".complete")
    if not os.path.exists(done):
        _say(f"writing random bf16 weights to {d}")
        t0 = time.time()
        shutil.rmtree(d, ignore_errors=True)
        cfg = dict(config)
        cfg.pop("head_dim", None)          # the reference computes it and refuses nothing, but keep to its own keys
        write_random_model(d, cfg, seed, torch.bfloat16)
        with open(done, "w") as f:
            f.write("ok\n")
        _say(f"written in {time.time() - t0:.0f} s")
    return d


def generate(binary: str, model_dir: str, ids, max_new: int, timeout: float) -> dict:
    """One run of the reference's command line; its JSON line as a dict, plus the wall time of the process."""
    ids_arg = ",".join(str(int(i)) for i in ids)
    t0 = time.time()
    try:
        r = subprocess.run([binary, model_dir, "--ids", ids_arg, "--max-new", str(max_new), "--ignore-eos", "--json",
                            "--kv-cache"], capture_output=True, text=True, timeout=max(timeout, 1.0))
    except subprocess.TimeoutExpired:
        raise Unavailable(f"a run of the reference ({len(ids)} prompt ids, {max_new} new) did not end within {timeout:.0f} s")
    if r.returncode != 0:
        raise Unavailable("llmi-generate failed: " + (r.stderr.strip().splitlines() or ["no message"])[-1][:200])
    out = json.loads(r.stdout.strip().splitlines()[-1])
    out["wall_seconds"] = time.time() - t0
    return out


def random_ids(n: int, vocab: int, seed: int):
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def run(config: dict, batch: int, context: int, prefill_tokens: int, steps: int, warmup: int, layers_full: int) -> dict:
    """The benchmark line of the reference arm (raises :class:`Unavailable` with what was measured so far)."""
    limit = float(os.environ.get("LLMI_REFERENCE_LIMIT_S", "1600"))
    t_start = time.time()
    left = lambda: limit - (time.time() - t_start)
    steps = max(steps, 128)           # fewer decode steps would drown in the run-to-run spread of the long prefills
    warmup = max(warmup, 3)
    binary = ensure_binary()
    model_dir = write_model(config)
    V = config["vocab_size"]
    partial = {}

    # 1. prefill of the benchmark's prompt; it also tells how fast this machine is
    p = generate(binary, model_dir, random_ids(prefill_tokens, V, 2), 1, left())
    prefill_s, load_s = p["generate_seconds"], p["load_seconds"]
    partial.update({"load_seconds": round(load_s, 2), "prefill_ms": round(prefill_s * 1e3, 1),
                    "prefill_tokens_per_s": round(prefill_tokens / prefill_s, 1)})
    _say(f"load {load_s:.1f} s; prefill of {prefill_tokens}: {prefill_s:.1f} s")
    prompt_len = context - warmup - steps
    # 2. what the two decode runs will cost: a prompt's products grow with its length and its attention with the
    # square of it (the reference's attention runs on one thread and is about half of the measured run's time at this
    # size, so the mean of the two growth rates is taken), and a decode step at the full context is taken as four
    # tokens' worth of the prompt's time
    scale = max(1.0, prompt_len / prefill_tokens)
    est = 2 * (load_s + prefill_s * (scale + scale * scale) / 2) + (2 * warmup + steps) * 4.0 * prefill_s / prefill_tokens
    partial["estimated_seconds_for_decode_runs"] = round(est)
    if est > left():
        raise Unavailable(f"the reference runs on the CPU: its two decode runs at context {context} are estimated at "
                          f"{est:.0f} s, over the {left():.0f} s left of its time limit (LLMI_REFERENCE_LIMIT_S={limit:.0f})",
                          partial)

    # 3. decode at the benchmark's context: the same prompt, ending `warmup` and `warmup + steps` tokens later
    ids = random_ids(prompt_len, V, 3)
    r1 = generate(binary, model_dir, ids, warmup, left())
    _say(f"{prompt_len} ids + {warmup} tokens: {r1['generate_seconds']:.1f} s")
    partial["seconds_prompt_and_warmup"] = round(r1["generate_seconds"], 2)
    r2 = generate(binary, model_dir, ids, warmup + steps, left())
    _say(f"{prompt_len} ids + {warmup + steps} tokens: {r2['generate_seconds']:.1f} s")
    if r2["generated_ids"][:warmup] != r1["generated_ids"]:
        raise Unavailable("two runs of the reference over the same prompt disagree on their first tokens", partial)
    ms_per_token = (r2["generate_seconds"] - r1["generate_seconds"]) / steps * 1e3
    if ms_per_token <= 0:
        raise Unavailable("the reference's two runs differ by less than their spread; no decode time", partial)
    value = 1000.0 / ms_per_token
    return {
        "metric": "decode tok/s at batch 8, context 4096 (SmolLM2-1.7B shape)", "value": round(value, 3), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(ms_per_token * batch, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp32 arithmetic on bf16-stored weights (the reference has no other compute type)",
        "data": "synthetic (random weights, uniform random token ids)", "impl": "reference",
        "config": {"model": "SmolLM2-1.7B shape", "layers": config["num_hidden_layers"], "layers_full": layers_full,
                   "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
                   "kv_heads": config["num_key_value_heads"], "head_dim": config["hidden_size"] // config["num_attention_heads"],
                   "intermediate": config["intermediate_size"], "vocab": V, "rope_theta": config["rope_theta"],
                   "rms_norm_eps": config["rms_norm_eps"], "tied": True, "global_batch": batch, "seq_len": context,
                   "prefill_tokens": prefill_tokens, "parallelism": "CPU, %d hardware threads" % (os.cpu_count() or 0),
                   "weights": "random bf16, widened to fp32 at load",
                   "batch": "%d sequences served one after another (the reference has no batching, src/server/server.cpp:44-50)" % batch,
                   "how": "llmi-generate --kv-cache --json: generate_seconds of two runs over one prompt, %d tokens apart" % steps},
        "e2e": {"value": round(value, 3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "note": "the reference has no device boundary: the same number"},
        "gpu_launches": 0,
        "prefill": {"value": round(prefill_tokens / prefill_s, 2), "tokens": prefill_tokens, "ms": round(prefill_s * 1e3, 1)},
        "points": {"decode_b1": round(value, 3)},
        "load_seconds": round(load_s, 2), "wall_seconds": round(time.time() - t_start, 1),
    }


def main(config: dict, batch: int, context: int, prefill_tokens: int, steps: int, warmup: int, layers_full: int) -> int:
    try:
        print(json.dumps(run(config, batch, context, prefill_tokens, steps, warmup, layers_full)))
    except Unavailable as e:
        line = {"impl": "reference", "unavailable": e.why}
        if e.partial:
            line["measured_before_giving_up"] = e.partial
        print(json.dumps(line))
    return 0
