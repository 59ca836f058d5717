"""Makes ``reference_tiny.npz``: outputs of the reference engine's own binary on two tiny models.

Run once, on a CPU, where the reference project's sources are available:

    python tests/golden/make_golden.py /path/to/llm-inference-cpp [build_dir]

It builds ``llmi-generate`` from those sources (cmake, tests off, no network needed), writes
two tiny model folders into a temporary folder with weights from an integer hash (exact on
every platform, no random-number library involved), runs
``llmi-generate DIR --ids ... --max-new 0 --dump FILE`` for the all-position logits and layer
states and ``--max-new 8 --ignore-eos --json [--kv-cache]`` for greedy ids, and stores the
results.  Two things the programs do not print come from ``reference_driver.cpp`` (beside this file),
which it compiles against the reference's ``libllmi.a``: the probabilities the reference's sampler draws
from (``llmi::sampling_probabilities``) for a few rows of logits under several settings, exact ties
included, and the logits of ``forward_cached`` fed in portions of several tokens (a sequence continued by
more than one token).  ``tests/test_plain_reference.py`` rebuilds the same folders with ``write_model``
below and checks the plain implementation (``tests/plain_llama.py``) against the stored outputs.
"""
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

CONFIGS = {
    "A": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
          "num_key_value_heads": 2, "intermediate_size": 176, "vocab_size": 256, "rope_theta": 10000.0,
          "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128, "hidden_act": "silu"},
    "B": {"architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 120, "num_attention_heads": 5,
          "num_key_value_heads": 1, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 100000.0,
          "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256, "hidden_act": "silu",
          "attention_bias": True},
}
PROMPTS = {"A": [5, 9, 1, 30, 7, 200, 13, 13, 77, 4, 0, 255, 31, 8, 100, 64, 2],
           "B": [383, 0, 17, 250, 3, 3, 99, 301, 12, 45, 7, 180, 222, 5, 64, 128, 19, 20, 21, 300, 1]}


def hashed_uniform(n: int, key: int) -> np.ndarray:
    """n numbers in [-1, 1) from splitmix64 of (key, index): integer arithmetic only."""
    with np.errstate(over="ignore"):
        x = np.arange(n, dtype=np.uint64) + np.uint64(key) * np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        x = x ^ (x >> np.uint64(31))
    return ((x >> np.uint64(40)).astype(np.float64) / float(1 << 23) - 1.0).astype(np.float32)


def tensor_table(cfg):
    """Tensor names and shapes in the reference's order (src/model/model.cpp:135-162)."""
    h, nh = cfg["hidden_size"], cfg["num_attention_heads"]
    hd = h // nh
    q, kv, ff, v = nh * hd, cfg["num_key_value_heads"] * hd, cfg["intermediate_size"], cfg["vocab_size"]
    out = [("model.embed_tokens.weight", (v, h))]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        out += [(p + "input_layernorm.weight", (h,)), (p + "self_attn.q_proj.weight", (q, h)),
                (p + "self_attn.k_proj.weight", (kv, h)), (p + "self_attn.v_proj.weight", (kv, h))]
        if cfg.get("attention_bias"):
            out += [(p + "self_attn.q_proj.bias", (q,)), (p + "self_attn.k_proj.bias", (kv,)),
                    (p + "self_attn.v_proj.bias", (kv,))]
        out += [(p + "self_attn.o_proj.weight", (h, q)), (p + "post_attention_layernorm.weight", (h,)),
                (p + "mlp.gate_proj.weight", (ff, h)), (p + "mlp.up_proj.weight", (ff, h)),
                (p + "mlp.down_proj.weight", (h, ff))]
    out.append(("model.norm.weight", (h,)))
    if not cfg.get("tie_word_embeddings"):
        out.append(("lm_head.weight", (v, h)))
    return out


def make_weights(cfg):
    w = {}
    for key, (name, shape) in enumerate(tensor_table(cfg)):
        u = hashed_uniform(int(np.prod(shape)), key + 1).reshape(shape)
        w[name] = (1.0 + 0.2 * u if name.endswith("norm.weight") else 0.15 * u).astype(np.float32)
    return w


def write_model(model_dir, name):
    """config.json + model.safetensors (F32) for golden configuration ``name``."""
    cfg = CONFIGS[name]
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    w = make_weights(cfg)
    header, off = {}, 0
    for n in sorted(w):
        nb = w[n].nbytes
        header[n] = {"dtype": "F32", "shape": list(w[n].shape), "data_offsets": [off, off + nb]}
        off += nb
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(os.path.join(model_dir, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for n in sorted(w):
            f.write(w[n].astype("<f4").tobytes())
    return cfg


# (temperature, top_k, top_p) settings for the sampler's probabilities; the reference's defaults are 1, 0, 1
SAMPLING = [(0.8, 0, 1.0), (1.0, 40, 1.0), (1.0, 0, 0.9), (0.7, 50, 0.95), (1.5, 3, 0.5), (0.0, 0, 1.0)]
PORTIONS = {"A": 5, "B": 7}


def sampling_rows(out):
    """Rows of logits for the sampler: real rows of both models (scaled up, so that top-p has something to cut)
    and made-up rows with exact ties — at the maximum, at the top-k border and inside the nucleus."""
    rows = {"A": out["A_logits"][[0, 7, 16]] * 8.0, "B": out["B_logits"][[1, 20]] * 8.0}
    ties = np.zeros((4, 16), dtype=np.float32)
    ties[0, [3, 9]] = 2.0                                   # two equal maxima
    ties[1] = np.repeat(np.arange(8, dtype=np.float32), 2)  # pairs of equal values everywhere
    ties[2, :] = 1.0                                        # all equal
    ties[3] = np.array([5, 5, 5, 1, 1, 1, 0, 0, -1, -1, -2, -2, -3, -3, -30, -30], dtype=np.float32)
    rows["ties"] = ties
    return rows


def main():
    src = sys.argv[1]
    build = sys.argv[2] if len(sys.argv) > 2 else tempfile.mkdtemp(prefix="llmi-build-")
    binary = os.path.join(build, "llmi-generate")
    if not os.path.exists(binary):
        subprocess.run(["cmake", "-S", src, "-B", build, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release",
                        "-DLLMI_BUILD_TESTS=OFF"], check=True)
        subprocess.run(["cmake", "--build", build, "--target", "llmi-generate"], check=True)
    here = os.path.dirname(os.path.abspath(__file__))
    driver = os.path.join(build, "reference_driver")
    subprocess.run(["cmake", "--build", build, "--target", "llmi"], check=True)
    subprocess.run(["g++", "-std=c++20", "-O2", "-I", os.path.join(src, "include"), os.path.join(here, "reference_driver.cpp"),
                    os.path.join(build, "libllmi.a"), "-lpthread", "-o", driver], check=True)
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for name in CONFIGS:
            d = os.path.join(tmp, name)
            write_model(d, name)
            ids = ",".join(map(str, PROMPTS[name]))
            dump = os.path.join(tmp, f"{name}.bin")
            subprocess.run([binary, d, "--ids", ids, "--max-new", "0", "--dump", dump], check=True)
            with open(dump, "rb") as f:
                head = json.loads(f.readline())
                data = np.frombuffer(f.read(), dtype="<f4")
            t, h, v, n = head["tokens"], head["hidden"], head["vocab"], head["states"]
            out[f"{name}_states"] = data[:n * t * h].reshape(n, t, h).copy()
            out[f"{name}_logits"] = data[n * t * h:].reshape(t, v).copy()
            for flag, key in (([], "greedy"), (["--kv-cache"], "greedy_cached")):
                r = subprocess.run([binary, d, "--ids", ids, "--max-new", "8", "--ignore-eos", "--json", *flag],
                                   check=True, capture_output=True, text=True)
                out[f"{name}_{key}"] = np.asarray(json.loads(r.stdout)["generated_ids"], dtype=np.int32)
            part = os.path.join(tmp, f"{name}_portions.f32")
            subprocess.run([driver, "portions", d, ids, str(PORTIONS[name]), part], check=True)
            out[f"{name}_portions_logits"] = np.fromfile(part, dtype="<f4").reshape(t, v).copy()
        for name, rows in sampling_rows(out).items():
            out[f"sampling_{name}_logits"] = rows
            fin = os.path.join(tmp, f"s_{name}.f32")
            rows.astype("<f4").tofile(fin)
            for i, (temp, k, p) in enumerate(SAMPLING):
                fout = os.path.join(tmp, f"s_{name}_{i}.f32")
                subprocess.run([driver, "sampling", fin, str(rows.shape[0]), str(rows.shape[1]), repr(temp), str(k),
                                repr(p), fout], check=True)
                out[f"sampling_{name}_{i}"] = np.fromfile(fout, dtype="<f4").reshape(rows.shape).copy()
    np.savez_compressed(os.path.join(here, "reference_tiny.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
