"""Recorded steps: one CUDA graph per (batch bucket, page-table bucket, choice) for decode steps, and one per
(token bucket, sequence bucket, wanted-rows bucket, page-table bucket) for short prompt steps.

A decode step of a small model is a few hundred short kernels; launched one by one from
Python, the launches cost more than the kernels.  A step's device work depends on the host
only through the index arrays of :mod:`batch` — and those live at fixed addresses in one
device block — so the whole step (embedding … head … choice of the next token) is recorded
once per shape and replayed: the host writes the index block, copies it, and launches one
graph.  Batches are padded up to a power of two of sequences and page tables to a power of
two of pages; padding sequences have index -1 and are skipped by every kernel, so padding
changes no result.  A graph holds raw addresses: it is keyed by the serial number of the
cache it was recorded for (never by the object's identity, which a later cache can get
again), it is not used once a scratch buffer it reads is reallocated
(``Runtime.generation``), and it is dropped when its cache dies.

One step ahead: between two decode steps the device would wait for the host to lay out the next index
block (about 80 us at batch 8, of a step of 1.8 ms).  So, right after a step is launched, the next one is
laid out as if the same sequences went on — positions reserved ahead in the cache, lengths and page tables
patched — while the device computes; when the caller comes back with exactly those sequences, only their
tokens are filled in and the block is uploaded.  If another step comes instead (a sequence ended, a prompt
in between), the reservation is taken back (``SequenceCache.settle``) and the step is planned the ordinary
way.  ``LLMI_AHEAD=0`` switches it off.

Prompt steps (:class:`PromptGraphs`).  A prompt of a few hundred tokens is bound by the host as well: about two
hundred launches of 6 to 15 us each, 2.9 ms whether the prompt has 16 or 256 tokens, where the device needs a
third of that.  Such steps are padded to a shape — token rows to 16, 32 or a multiple of 64 (128 from 512 on), sequences and
wanted rows to a power of two, page tables as for decode steps; the padding rows belong to no sequence — and a
shape that comes a second time is recorded and replayed from then on.  Prompts beyond 1,024 tokens keep the device
busy for longer than their launches take and run launch by launch, unpadded.
"""
from __future__ import annotations

import os
import weakref

import torch

# LLMI_GRAPHS=0 runs every decode step launch by launch (for profilers that want single kernels).
RECORD = os.environ.get("LLMI_GRAPHS", "1") != "0"
# LLMI_AHEAD=0: never lay the next decode step out ahead of its tokens.
AHEAD = os.environ.get("LLMI_AHEAD", "1") != "0"


def bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


def _drop_graphs_of(graphs_ref, serial: int) -> None:
    graphs = graphs_ref()
    if graphs is not None:
        graphs._drop_cache(serial)


class DecodeGraphs:
    def __init__(self, model):
        self.model = model
        self.graphs = {}
        self.replays = 0
        self.kernels_per_graph = {}
        self._last = None        # (weak cache, page bucket, context, buffer identity) of the step before
        self._watched = set()    # serials of the caches whose death drops their graphs
        self._pending = None     # (weak cache, page bucket, context, PendingStep, buffer identity): the next step, laid out ahead
        self.ahead_used = 0      # steps that were laid out ahead and then came

    def _drop_cache(self, serial: int) -> None:
        for key in [k for k in self.graphs if k[3] == serial]:
            del self.graphs[key]
            self.kernels_per_graph.pop(key, None)
        self._watched.discard(serial)
        if self._last is not None and self._last[0]() is None:
            self._last = None        # its context holds the dead cache's groups

    def _key(self, B, P, choice, cache, plan=()):
        m = self.model
        return (B, P, choice, cache.serial, m.rt.generation, m.buffers.dev.data_ptr(), plan)

    def step(self, cache, seqs, sampler, streams=None):
        """A decode step (one token per sequence) followed by the choice; returns device int32 ids
        of the real sequences (valid until the next step)."""
        from .batch import continue_decode_step, finish_continue, plan_step
        m = self.model
        n_real = len(seqs)
        B = bucket(n_real)
        ctx = None
        pend, self._pending = self._pending, None
        if pend is not None:
            p_cache, P, p_ctx, p_step, p_ident = pend
            if (p_cache() is cache and p_ctx.layout.slots == tuple(s.slot for s in seqs) and cache.slots.all_live(p_ctx.layout.slots)
                    and p_ident == (m.rt.generation, m.buffers.dev.data_ptr(), m.buffers.serial)):
                # the step that was laid out ahead has come: its tokens, one upload
                finish_continue(cache, p_ctx, p_step, [s.tokens[0] for s in seqs], m.spec.vocab_size, m.buffers)
                ctx = p_ctx
                self.ahead_used += 1
            elif p_cache() is not None:
                p_cache().settle()
        last = self._last if ctx is None else None
        if last is not None:
            l_cache, P, l_ctx, l_ident = last
            slots = l_ctx.layout.slots
            if (l_cache() is cache and slots == tuple(s.slot for s in seqs) and cache.slots.all_live(slots)
                    and l_ident == (m.rt.generation, m.buffers.dev.data_ptr(), m.buffers.serial)
                    and (max(cache.length(s) for s in slots) + cache.page_size) // cache.page_size <= P):
                # the same sequences one token on, and nobody used the index block in between:
                # patch the step before instead of planning anew
                continue_decode_step(cache, l_ctx, [s.tokens[0] for s in seqs], m.spec.vocab_size, m.buffers)
                ctx = l_ctx
        if ctx is None:
            self._last = None
            need_pages = max((cache.length(s.slot) + 1 + cache.page_size - 1) // cache.page_size for s in seqs)
            P = max(need_pages, min(bucket(need_pages), cache.max_pages_per_seq))
            ctx = plan_step(cache, seqs, m.spec.vocab_size, m.buffers, pad_seqs_to=B, pad_pages_to=P)
        self._last = (weakref.ref(cache), P, ctx, (m.rt.generation, m.buffers.dev.data_ptr(), m.buffers.serial))
        m._last_h2d = ctx.h2d_bytes
        sampler.prepare(B, streams)
        choice = (sampler.params.temperature, sampler.params.top_k, sampler.params.top_p)
        plan = m.step_plan_token(ctx, cache)      # (a decode kernel's split follows the live sequences)
        key = self._key(B, P, choice, cache, plan)
        entry = self.graphs.get(key)
        if entry is None:
            # first time for this shape: run it plainly (this also sizes every scratch buffer), then record
            logits = m.run(ctx, cache)
            ids = sampler.launch(logits, B)
            m.last_logits = logits[:n_real]
            key = self._key(B, P, choice, cache, plan)     # the plain run may have grown a scratch buffer
            if RECORD and key not in self.graphs:
                # graphs of shapes recorded before a buffer moved can never be replayed again
                for stale in [k for k in self.graphs if k[3] == cache.serial and k[4:6] != key[4:6]]:
                    del self.graphs[stale]
                    self.kernels_per_graph.pop(stale, None)
                if cache.serial not in self._watched:
                    self._watched.add(cache.serial)
                    weakref.finalize(cache, _drop_graphs_of, weakref.ref(self), cache.serial)
                from ..ops import kernels
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                before = kernels.launch_count()
                with torch.cuda.graph(g):
                    rec_logits = m.run(ctx, cache)
                    rec_ids = sampler.launch(rec_logits, B)
                self.kernels_per_graph[key] = kernels.launch_count() - before
                kernels.launch_count(-(kernels.launch_count() - before))   # recording launches nothing
                self.graphs[key] = (g, rec_ids, rec_logits)
            self._lay_out_next(cache, ctx, P)
            return ids[:n_real]
        g, rec_ids, rec_logits = entry
        g.replay()
        m.last_logits = rec_logits[:n_real]
        self.replays += 1
        from ..ops import kernels
        kernels.launch_count(self.kernels_per_graph[key])
        self._lay_out_next(cache, ctx, P)
        return rec_ids[:n_real]

    def _lay_out_next(self, cache, ctx, P) -> None:
        """While the device runs the step just launched: the next step's block, as if the same sequences went on."""
        if not AHEAD or not cache.can_speculate():
            return
        from ..cache.pages import CacheError
        from .batch import prepare_continue
        slots = ctx.layout.slots
        if (max(cache.length(s) for s in slots) + cache.page_size) // cache.page_size > P:
            return                              # the page tables would outgrow this shape: the next step is planned anew
        m = self.model
        try:
            step = prepare_continue(cache, ctx, m.buffers)
        except CacheError:
            return                              # no room (or the context's end): whatever comes next will say so
        self._pending = (weakref.ref(cache), P, ctx, step, (m.rt.generation, m.buffers.dev.data_ptr(), m.buffers.serial))


def prompt_bucket(n_tokens: int) -> int:
    """The padded number of token rows of a prompt step, 0 if such a step is not padded (and not recorded)."""
    if n_tokens <= 32:
        return 16 if n_tokens <= 16 else 32          # the weight-streaming products' range
    if n_tokens <= 512:
        return (n_tokens + 63) // 64 * 64
    if n_tokens <= 1024:
        return (n_tokens + 127) // 128 * 128
    return 0


class PromptGraphs:
    """Prompt steps by shape: padded, run plainly the first time a shape comes, recorded the second time, replayed after."""
    MAX_GRAPHS = 96          # per model; the oldest shapes go first

    def __init__(self, model):
        self.model = model
        self.graphs = {}         # key -> (graph, logits, kernels launched)
        self.seen = {}           # key -> times the shape has come without a graph
        self.replays = 0
        self._watched = set()

    def _drop_cache(self, serial: int) -> None:
        for table in (self.graphs, self.seen):
            for key in [k for k in table if k[4] == serial]:
                del table[key]
        self._watched.discard(serial)

    def _key(self, T, S, W, P, cache):
        m = self.model
        return (T, S, W, P, cache.serial, m.rt.generation, m.buffers.dev.data_ptr())

    def step(self, cache, seqs):
        """fp32 logits [wanted, vocab] of a prompt step (scratch: valid until the next step), or None if the step
        is not one for this path (too long): the caller then runs it the plain way."""
        from .batch import plan_step
        from ..ops import kernels
        m = self.model
        T = prompt_bucket(sum(len(s.tokens) for s in seqs))
        if T == 0:
            return None
        S = bucket(len(seqs))
        n_want_real = sum(len(s.want) for s in seqs)
        W = bucket(n_want_real) if n_want_real else 0
        ps = cache.page_size
        # (a slot that is not live, or a step that does not fit, is plan_step's to report)
        try:
            need_pages = max((cache.length(s.slot) + len(s.tokens) + ps - 1) // ps for s in seqs)
        except Exception:
            need_pages = 1
        P = max(need_pages, min(bucket(need_pages), cache.max_pages_per_seq))
        ctx = plan_step(cache, seqs, m.spec.vocab_size, m.buffers, pad_seqs_to=S, pad_pages_to=P, pad_tokens_to=T, pad_want_to=W)
        m._last_h2d = ctx.h2d_bytes
        key = self._key(T, S, W, P, cache)
        entry = self.graphs.get(key)
        if entry is not None:
            g, rec_logits, n_kernels = entry
            g.replay()
            self.replays += 1
            kernels.launch_count(n_kernels)
            return rec_logits[:n_want_real]
        logits = m.run(ctx, cache)
        key = self._key(T, S, W, P, cache)          # the plain run may have grown a scratch buffer
        self.seen[key] = self.seen.get(key, 0) + 1
        if RECORD and self.seen[key] >= 2:
            for table in (self.graphs, self.seen):   # shapes recorded or counted before a buffer moved never come again
                for stale in [k for k in table if k[4] == cache.serial and k[5:] != key[5:]]:
                    del table[stale]
            while len(self.graphs) >= self.MAX_GRAPHS:
                del self.graphs[next(iter(self.graphs))]
            if cache.serial not in self._watched:
                self._watched.add(cache.serial)
                weakref.finalize(cache, _drop_graphs_of, weakref.ref(self), cache.serial)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before = kernels.launch_count()
            with torch.cuda.graph(g):
                rec_logits = m.run(ctx, cache)
            n_kernels = kernels.launch_count() - before
            kernels.launch_count(-n_kernels)          # recording launches nothing
            self.graphs[key] = (g, rec_logits, n_kernels)
            self.seen.pop(key, None)
        return logits[:n_want_real]
