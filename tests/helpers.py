"""Helpers of the replay tests: building traces in the three ways of cutting, and collecting logits."""
import numpy as np

PAGE = 64


def rel_to_max(a, b):
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - b)) / max(float(np.max(np.abs(b))), 1e-30))


# Tolerances, set once: the engine's fp32 path against the float64 plain implementation, and the
# bf16 path (bf16 weights, activations and cache; fp32 accumulation) against the same.
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def round_up(n, m=PAGE):
    return (n + m - 1) // m * m


def trace_whole(requests):
    """Each request alone and whole.  requests: {id: tokens}."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps, max(round_up(len(t)) for t in requests.values())


def trace_last_decoded(requests, n_last=32):
    """Each request alone: all but the last ``n_last`` tokens in one step, then one token a step."""
    steps, k = [], 0
    for rid, toks in requests.items():
        cut = max(1, len(toks) - n_last)
        steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[:cut], "want": list(range(cut))}],
                      "end": [rid] if cut == len(toks) else []})
        k += 1
        for t in range(cut, len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[t]], "want": [0]}],
                          "end": [rid] if t == len(toks) - 1 else []})
            k += 1
    return steps, max(round_up(len(t)) for t in requests.values())


def trace_batches(requests, batch_size, prompt_lens):
    """Batches of unequal lengths, one after another: the requests of a batch start together with
    prompts of ``prompt_lens[id]`` tokens, then go on by one token each; shorter ones end earlier."""
    ids = list(requests)
    steps, k, most = [], 0, 0
    for b in range(0, len(ids), batch_size):
        batch = ids[b:b + batch_size]
        most = max(most, sum(round_up(len(requests[r])) for r in batch))
        fed = {r: min(prompt_lens[r], len(requests[r])) for r in batch}
        entries = [{"id": r, "tokens": requests[r][:fed[r]], "want": list(range(fed[r]))} for r in batch]
        live = list(batch)
        while entries:
            ending = [r for r in live if fed[r] == len(requests[r])]
            steps.append({"step": k, "entries": entries, "end": ending})
            k += 1
            live = [r for r in live if r not in ending]
            entries = []
            for r in live:
                entries.append({"id": r, "tokens": [requests[r][fed[r]]], "want": [0]})
                fed[r] += 1
    return steps, most


def trace_portions(requests, portion, n_last=4):
    """Each request alone: its tokens but the last ``n_last`` in portions of ``portion`` tokens (the last portion is
    what is left), then one token a step — a prompt fed in parts, as a chat's next turn continues a sequence."""
    steps, k = [], 0
    for rid, toks in requests.items():
        cut = max(1, len(toks) - n_last)
        for a in range(0, cut, portion):
            b = min(a + portion, cut)
            steps.append({"step": k, "entries": [{"id": rid, "tokens": toks[a:b], "want": list(range(b - a))}],
                          "end": [rid] if b == len(toks) else []})
            k += 1
        for t in range(cut, len(toks)):
            steps.append({"step": k, "entries": [{"id": rid, "tokens": [toks[t]], "want": [0]}],
                          "end": [rid] if t == len(toks) - 1 else []})
            k += 1
    return steps, max(round_up(len(t)) for t in requests.values())


def trace_mixed(requests, first, portion):
    """All requests in one batch: request r starts with ``first[r]`` tokens and then goes on by ``portion[r]`` tokens a
    step (1: it decodes) until it ends — steps in which some sequences continue a prompt and others decode."""
    ids = list(requests)
    fed = {r: 0 for r in ids}
    steps, k, live = [], 0, list(ids)
    while live:
        entries = []
        for r in live:
            n = min(first[r] if fed[r] == 0 else portion[r], len(requests[r]) - fed[r])
            entries.append({"id": r, "tokens": requests[r][fed[r]:fed[r] + n], "want": list(range(n))})
            fed[r] += n
        ending = [r for r in live if fed[r] == len(requests[r])]
        steps.append({"step": k, "entries": entries, "end": ending})
        k += 1
        live = [r for r in live if r not in ending]
    return steps, sum(round_up(len(t)) for t in requests.values())


def collect(steps, outputs, vocab):
    """{id: [T, vocab]} from the per-step outputs of a replay (None where nothing was wanted)."""
    rows = {}
    for step, out in zip(steps, outputs):
        off = 0
        for e in step["entries"]:
            for _ in e["want"]:
                rows.setdefault(e["id"], []).append(out[off])
                off += 1
        assert out is None or off == out.shape[0]
    return {r: np.stack(v).reshape(-1, vocab) for r, v in rows.items()}


def replay(model, steps, max_tokens, poison=True):
    """Run a trace in-process through the library's TraceReplayer; returns the per-step logits."""
    import torch
    from llmi_b200.engine.trace import TraceReplayer
    rp = TraceReplayer(model, max_tokens)
    if poison:      # whatever is read outside a sequence's own positions turns the logits to NaN
        for g in rp.cache.kv_groups:
            g.k.fill_(float("nan"))
            g.v.fill_(float("nan"))
    outs = []
    for s in steps:
        o = rp.run_step(s)
        outs.append(None if o is None else o.copy())
    rp.cache.check()
    assert not rp.slots and not rp.cache.slots.live
    for g in rp.cache.kv_groups:
        assert g.pool.n_free == g.pool.n_pages
    torch.cuda.synchronize()
    return outs
