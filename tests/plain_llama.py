"""A plain, slow implementation of the Llama / SmolLM2 decoder: the oracle of the tests.

Whole sequences, no cache, no batching, one function for each part, numpy only.
It shares no code with the library (it even reads model folders with its own few
lines).  Each function restates a formula of the reference engine and cites it by
file:line within fernandojcardenas/llm-inference-cpp.  ``tests/golden/`` holds
outputs of the reference's own binary on a tiny random model, and
``tests/test_plain_reference.py`` checks this file against them, so the oracle does
not rest on the formulas alone.

Arithmetic is float64 by default (``dtype=np.float64``): the library's fp32 and
bf16 results are then compared against something more exact than either.  With
``dtype=np.float32`` it follows the reference's own precision.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np


# ----------------------------------------------------------------------------- model folder

def read_safetensors(path):
    """name -> float64 array.  Format: src/model/safetensors.cpp:116-223; BF16 widening by
    ``bits << 16``: src/model/safetensors.cpp:276-299."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        raw = data[a:b]
        if e["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif e["dtype"] == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        else:
            raise ValueError(f"plain reader: dtype {e['dtype']} of {name}")
        out[name] = arr.reshape(e["shape"])
    return out


def read_model(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


def sizes(cfg):
    """The numbers the forward pass needs, from config.json keys (src/model/model.cpp:84-107)."""
    nh = cfg["num_attention_heads"]
    return dict(L=cfg["num_hidden_layers"], H=cfg["hidden_size"], nh=nh,
                nkv=cfg.get("num_key_value_heads") or nh,
                hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
                F=cfg["intermediate_size"], V=cfg["vocab_size"], eps=cfg["rms_norm_eps"], theta=cfg["rope_theta"],
                tied=bool(cfg.get("tie_word_embeddings", False)), bias=bool(cfg.get("attention_bias", False)))


# ----------------------------------------------------------------------------- the parts

def embedding(table, tokens):
    """x[t, :] = E[token[t], :], no scaling (src/model/transformer.cpp:97-100)."""
    return table[np.asarray(tokens)]


def rmsnorm(x, weight, eps):
    """y = w * (x * scale), scale = 1/sqrt(mean(x^2) + eps); eps first rounded to float
    (src/model/kernels.cpp:115-120; src/model/transformer.cpp:89)."""
    eps = float(np.float32(eps))
    scale = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return weight * (x * scale)


def linear(x, w, bias=None):
    """y[r, o] = dot(x[r], w[o]) + bias[o], w is [out, in] (src/model/kernels.cpp:97-113)."""
    y = x @ w.T
    return y if bias is None else y + bias


def rope_inv_freq(head_dim, theta):
    """inv_freq[i] = 1 / theta^(2i/d) computed in float32 (src/model/transformer.cpp:59-65)."""
    i = np.arange(head_dim // 2)
    exponent = (2 * i).astype(np.float32) / np.float32(head_dim)
    return (np.float32(1.0) / np.power(np.float32(theta), exponent)).astype(np.float32)


def rope(v, positions, inv_freq):
    """Rotate-half pairing (i, i + d/2); angle = float(pos) * inv_freq[i] as a float32 product
    (src/model/kernels.cpp:122-134).  v: [T, heads, d]."""
    half = v.shape[-1] // 2
    angle = (np.asarray(positions, dtype=np.float32)[:, None] * inv_freq[None, :]).astype(np.float32)
    c = np.cos(angle.astype(np.float64))[:, None, :].astype(v.dtype)
    s = np.sin(angle.astype(np.float64))[:, None, :].astype(v.dtype)
    a, b = v[..., :half], v[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def softmax(x):
    """exp(x - max) / sum (src/model/kernels.cpp:136-146)."""
    e = np.exp(x - np.max(x))
    return e / np.sum(e)


def attention(q, k, v, window=0):
    """Causal grouped-query attention on whole sequences.  q: [T, nh, d], k, v: [T, nkv, d].
    kv head = hh / (nh/nkv) (integer division); score = dot * (1/sqrt(d)) for s <= t
    (src/model/transformer.cpp:127-141).  ``window`` > 0 keeps keys t-window+1..t (the
    reference has no window; the library's mixer has the parameter)."""
    T, nh, d = q.shape
    group = nh // k.shape[1]
    scale = 1.0 / np.sqrt(np.float32(d)).astype(q.dtype)
    out = np.zeros_like(q)
    for hh in range(nh):
        kvh = hh // group
        for t in range(T):
            lo = max(0, t - window + 1) if window > 0 else 0
            scores = (k[lo:t + 1, kvh] @ q[t, hh]) * scale
            p = softmax(scores)
            out[t, hh] = p @ v[lo:t + 1, kvh]
    return out


def silu(z):
    """z / (1 + exp(-z)) (src/model/kernels.cpp:148)."""
    return z / (1.0 + np.exp(-z))


def swiglu_ffn(h, w_gate, w_up, w_down):
    """(silu(h Wg^T) * (h Wu^T)) Wd^T (src/model/transformer.cpp:149-152)."""
    return linear(silu(linear(h, w_gate)) * linear(h, w_up), w_down)


def attention_block(x, w, prefix, sz, positions, inv_freq):
    """RMSNorm, q/k/v projections (+bias), RoPE on q and k, attention, output projection
    (src/model/transformer.cpp:119-145)."""
    T = x.shape[0]
    h = rmsnorm(x, w[prefix + "input_layernorm.weight"], sz["eps"])
    bias = (lambda n: w[prefix + f"self_attn.{n}_proj.bias"]) if sz["bias"] else (lambda n: None)
    q = linear(h, w[prefix + "self_attn.q_proj.weight"], bias("q")).reshape(T, sz["nh"], sz["hd"])
    k = linear(h, w[prefix + "self_attn.k_proj.weight"], bias("k")).reshape(T, sz["nkv"], sz["hd"])
    v = linear(h, w[prefix + "self_attn.v_proj.weight"], bias("v")).reshape(T, sz["nkv"], sz["hd"])
    q, k = rope(q, positions, inv_freq), rope(k, positions, inv_freq)
    a = attention(q, k, v).reshape(T, sz["nh"] * sz["hd"])
    return linear(a, w[prefix + "self_attn.o_proj.weight"])


def decoder_layer(x, w, i, sz, positions, inv_freq):
    """x += attention(norm(x)); x += ffn(norm(x)) (include/llmi/model/transformer.hpp:49-52)."""
    p = f"model.layers.{i}."
    x = x + attention_block(x, w, p, sz, positions, inv_freq)
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], sz["eps"])
    return x + swiglu_ffn(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def forward(cfg, w, tokens, dtype=np.float64, return_states=False, rows=None):
    """Logits at every position of one whole sequence, [T, V] (src/model/transformer.cpp:78-166).
    ``return_states``: also embeddings, each layer's output and the final norm
    (include/llmi/model/transformer.hpp:14-16).  ``rows``: the head for these positions only (the
    reference's last-position mode, src/model/transformer.cpp:161-165, for any positions)."""
    sz = sizes(cfg)
    w = {k: v.astype(dtype) for k, v in w.items()}
    positions = np.arange(len(tokens))
    inv_freq = rope_inv_freq(sz["hd"], sz["theta"])
    x = embedding(w["model.embed_tokens.weight"], tokens)
    states = [x]
    for i in range(sz["L"]):
        x = decoder_layer(x, w, i, sz, positions, inv_freq)
        states.append(x)
    h = rmsnorm(x, w["model.norm.weight"], sz["eps"])
    states.append(h)
    head = w["model.embed_tokens.weight"] if sz["tied"] else w["lm_head.weight"]
    logits = linear(h if rows is None else h[np.asarray(rows)], head)
    return (logits, states) if return_states else logits


# ----------------------------------------------------------------------------- choosing tokens

def argmax(x):
    """First maximum (src/model/transformer.cpp:22-24)."""
    return int(np.argmax(x))


def sampling_probabilities(logits, temperature, top_k=0, top_p=1.0):
    """softmax(logits/T), top-k, then top-p on the descending order with ties by lower id,
    renormalised (src/model/sampling.cpp:11-58)."""
    logits = np.asarray(logits, dtype=np.float64)
    n = logits.shape[0]
    if temperature <= 0:
        p = np.zeros(n)
        p[argmax(logits)] = 1.0
        return p
    p = softmax(logits.astype(np.float32).astype(np.float64) / np.float64(np.float32(temperature)))
    p = p.astype(np.float32).astype(np.float64)
    order = np.argsort(-p, kind="stable")
    k = n if (top_k == 0 or top_k > n) else top_k
    keep = k
    if top_p < 1.0:
        cum = 0.0
        for i in range(k):
            cum += p[order[i]]
            if cum >= float(np.float32(top_p)):
                keep = i + 1
                break
        keep = max(1, min(keep, k))
    out = np.zeros(n)
    out[order[:keep]] = p[order[:keep]]
    return out / out.sum()


def sample(logits, temperature, top_k, top_p, u):
    """Inverse CDF in ascending id order: first id whose running sum reaches u
    (src/model/sampling.cpp:60-76)."""
    if temperature <= 0:
        return argmax(logits)
    p = sampling_probabilities(logits, temperature, top_k, top_p)
    cum = np.cumsum(p)
    idx = np.nonzero((cum >= u) & (p > 0))[0]
    return int(idx[0]) if len(idx) else int(np.nonzero(p > 0)[0][-1])


def generate_greedy(cfg, w, prompt, max_new, stop_ids=(), dtype=np.float64):
    """Recompute-everything greedy loop; the stop token is kept in the output
    (src/model/transformer.cpp:168-180)."""
    tokens, out = list(prompt), []
    for _ in range(max_new):
        nxt = argmax(forward(cfg, w, tokens, dtype)[-1])
        out.append(nxt)
        tokens.append(nxt)
        if nxt in stop_ids:
            break
    return out
