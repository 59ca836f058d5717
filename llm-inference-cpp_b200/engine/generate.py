"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early.

Per sequence the loop is the reference's cached greedy loop (src/model/transformer.cpp:308-327):
prefill, choose; then repeat { emit the token; stop if it is a stop token (the stop token is
kept in the output); stop at ``max_new``; feed it forward; choose }.  The last token is never
fed forward.  Stop ids default to the configuration's ``eos_token_id`` and are empty with
``ignore_eos`` (apps/llmi-generate/main.cpp:330-332).

What is new is the batch: the prompts of a batch run in one step, then every live sequence
advances by one token per step; a sequence that ends leaves the batch at once and its slot
and pages go back to the cache; nothing joins a running batch; requests that do not fit
wait for the next batch.  The decisions live in :func:`run_batches`, which only talks to a
*backend* (alloc / free / step-and-choose), so they can be tested without a device.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

from ..cache.pages import PAGE_SIZE, pages_for
from ..sampling import Sampler, SamplingParams, UniformStream
from .batch import SequenceStep


@dataclass
class Request:
    index: int
    prompt: list
    max_new: int
    output: list = field(default_factory=list)
    finish: str = ""            # "stop" | "length"


def plan_batches(requests, max_batch: int, max_tokens: int, page_size: int = PAGE_SIZE):
    """Split requests, in order, into batches that fit ``max_batch`` sequences and ``max_tokens``
    cache tokens (each request counted at its longest, rounded up to whole pages)."""
    batches, cur, used = [], [], 0
    for r in requests:
        need = pages_for(len(r.prompt) + max(r.max_new - 1, 0), page_size) * page_size
        if need > max_tokens:
            raise ValueError(f"request {r.index} needs {need} cache tokens; the cache holds {max_tokens}")
        if cur and (len(cur) >= max_batch or used + need > max_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(r)
        used += need
    if cur:
        batches.append(cur)
    return batches


def run_batches(batches, backend, stop_ids=()):
    """Drive ``backend`` through the batches; fills each request's ``output`` and ``finish``.

    backend.alloc() -> slot; backend.free(slot); backend.step(entries) -> chosen token per entry,
    where entries is a list of (slot, request, tokens to feed).
    Returns the number of steps run.
    """
    stop = set(int(s) for s in stop_ids)
    steps = 0
    for batch in batches:
        live = [(backend.alloc(), r) for r in batch if r.max_new > 0]
        for r in batch:
            if r.max_new <= 0:
                r.finish = "length"
        feed = [(slot, r, list(r.prompt)) for slot, r in live]
        while feed:
            chosen = backend.step(feed)
            steps += 1
            nxt = []
            for (slot, r, _), tok in zip(feed, chosen):
                tok = int(tok)
                r.output.append(tok)
                if tok in stop:
                    r.finish = "stop"
                elif len(r.output) >= r.max_new:
                    r.finish = "length"
                if r.finish:
                    backend.free(slot)
                else:
                    nxt.append((slot, r, [tok]))
            feed = nxt
    return steps


class ModelBackend:
    """run_batches' backend on a real model: step, choose on the device, read the ids back."""

    def __init__(self, model, cache, sampling: SamplingParams, use_graphs: bool = True):
        self.model, self.cache = model, cache
        self.sampler = Sampler(sampling, model.rt)
        self.sampling = sampling
        self.streams = {}
        self.use_graphs = use_graphs
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def alloc(self):
        return self.cache.alloc_slot()

    def free(self, slot):
        self.cache.free_slot(slot)

    def step(self, entries):
        seqs = [SequenceStep(slot, toks, [len(toks) - 1]) for slot, _, toks in entries]
        streams = None
        if not self.sampling.greedy:
            streams = []
            for _, r, _ in entries:
                if r.index not in self.streams:
                    self.streams[r.index] = UniformStream(self.sampling.seed, r.index)
                streams.append(self.streams[r.index])
        ids = self.model.step_and_choose(self.cache, seqs, self.sampler, streams, use_graphs=self.use_graphs)
        self.h2d_bytes += self.model.last_h2d_bytes
        self.d2h_bytes += ids.numel() * 4
        return ids.tolist()


def generate(model, prompts, max_new=32, stop_ids=None, ignore_eos: bool = False,
             sampling: SamplingParams | None = None, max_batch: int = 64, cache=None, max_tokens: int | None = None,
             use_graphs: bool = True, return_details: bool = False):
    """Generate for a list of prompts (lists of token ids).  Returns one list of new ids per prompt.

    ``max_new`` is one number or one per prompt.  ``stop_ids=None`` takes the configuration's end
    tokens; ``ignore_eos`` empties them.  ``cache`` reuses a cache of this model; otherwise one is
    made for ``max_tokens`` (default: what the largest batch needs).
    """
    sampling = sampling or SamplingParams()
    per = list(max_new) if isinstance(max_new, (list, tuple)) else [int(max_new)] * len(prompts)
    if len(per) != len(prompts):
        raise ValueError("generate: max_new must be one number or one per prompt")
    for p in prompts:
        if len(p) == 0:
            raise ValueError("generate: empty prompt")
    requests = [Request(i, [int(t) for t in p], int(n)) for i, (p, n) in enumerate(zip(prompts, per))]
    if stop_ids is None:
        stop_ids = () if ignore_eos else tuple(model.spec.stop_ids)
    elif ignore_eos:
        stop_ids = ()
    page = PAGE_SIZE
    if cache is None:
        if max_tokens is None:
            needs = sorted((pages_for(len(r.prompt) + max(r.max_new - 1, 0), page) * page for r in requests), reverse=True)
            max_tokens = max(page, sum(needs[:max_batch]))
        cache = model.new_cache(max_tokens)
    else:
        max_tokens = cache.kv_groups[0].pool.n_pages * cache.page_size if cache.kv_groups else 1 << 30
    batches = plan_batches(requests, max_batch, max_tokens, page)
    backend = ModelBackend(model, cache, sampling, use_graphs)
    t0 = time.perf_counter()
    steps = run_batches(batches, backend, stop_ids)
    seconds = time.perf_counter() - t0
    outputs = [r.output for r in requests]
    if return_details:
        return outputs, {"steps": steps, "seconds": seconds, "finish": [r.finish for r in requests],
                         "batches": len(batches), "h2d_bytes": backend.h2d_bytes, "d2h_bytes": backend.d2h_bytes}
    return outputs
