"""A step's batch: validation on the host, and the index arrays the kernels read.

One step runs the next tokens of some sequences — all at their first token, with
unequal lengths (prompts), or all continuing by one token (decode).  The reference's
step takes one sequence (src/model/transformer.cpp:192-212); its checks are kept per
sequence: no tokens, id out of range, cache full, context exceeded — plus a slot named
twice.  Tokens are flattened in sequence order; each token carries the index of its
sequence and its absolute position, and every cache group gets the page table of the
step's sequences.  All of it travels to the device as one int32 block in one copy.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.pages import CacheError, pages_for


class StepError(ValueError):
    pass


@dataclass
class SequenceStep:
    """The next tokens of one live sequence and the places among them whose logits are wanted."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


class StepBuffers:
    """Pinned host blocks and a device twin for the index arrays of steps; grow on demand.

    Two host blocks alternate, each guarded by an event, so that writing the next step's
    arrays never overtakes a copy that is still queued on the stream.
    """

    def __init__(self, device, rt=None):
        self.device = device
        self.rt = rt
        self.hosts = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.dev = None

    def stage(self, n_int32: int):
        """-> (host block to fill, device block); call ``upload`` when the host block is filled."""
        self.turn ^= 1
        i = self.turn
        if self.events[i] is not None:
            self.events[i].synchronize()
        if self.hosts[i] is None or self.hosts[i].numel() < n_int32:
            self.hosts[i] = torch.empty(max(4096, 2 * n_int32), dtype=torch.int32, pin_memory=True)
        if self.dev is None or self.dev.numel() < n_int32:
            self.dev = torch.empty(max(4096, 2 * n_int32), dtype=torch.int32, device=self.device)
            if self.rt is not None:
                self.rt.generation += 1
        return self.hosts[i], self.dev

    def upload(self, n_int32: int) -> None:
        i = self.turn
        self.dev[:n_int32].copy_(self.hosts[i][:n_int32], non_blocking=True)
        if self.events[i] is None:
            self.events[i] = torch.cuda.Event()
        self.events[i].record()


class StepContext:
    """Device views of one step's index arrays (see module docstring) and its host-side sizes."""

    def __init__(self):
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.max_q_len = self.max_kv_len = 0
        self.decode = False
        self.token_ids = self.tok_seq = self.tok_pos = self.want_rows = None
        self.seq_q_start = self.seq_kv_len = self.seq_slot = None
        self._pages = {}
        self.h2d_bytes = 0

    def pages_of(self, group) -> torch.Tensor:
        """[n_seqs, pages] int32 page table of this step's sequences in a cache group."""
        return self._pages[id(group)]


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


def plan_step(cache, seqs, vocab_size: int, buffers: StepBuffers, pad_seqs_to: int = 0,
              pad_pages_to: int = 0) -> StepContext:
    """Validate a step, reserve its cache room, and upload its index arrays.

    ``pad_seqs_to`` / ``pad_pages_to`` round the decode batch and the page tables up (padding
    sequences have index -1 and are skipped by every kernel) so that recorded launches of one
    shape can be replayed for smaller batches.
    """
    if not seqs:
        raise StepError("step: no sequences")
    seen = set()
    for s in seqs:
        if len(s.tokens) == 0:
            raise StepError("step: a sequence brings no tokens")
        if s.slot in seen:
            raise StepError(f"step: slot {s.slot} is named twice")
        seen.add(s.slot)
        for tok in s.tokens:
            if not (0 <= int(tok) < vocab_size):
                raise StepError(f"step: token id {tok} out of range")
        for w in s.want:
            if not (0 <= int(w) < len(s.tokens)):
                raise StepError(f"step: wanted place {w} is not among the {len(s.tokens)} tokens given")
    bases = [cache.length(s.slot) for s in seqs]          # raises CacheError for a slot that is not live
    firsts = [b == 0 for b in bases]
    decode = all(len(s.tokens) == 1 for s in seqs)
    if not decode and not all(firsts):
        raise StepError("step: sequences must all start at their first token or all continue by one token")
    cache.can_extend({s.slot: len(s.tokens) for s in seqs})
    for s in seqs:
        cache.extend(s.slot, len(s.tokens))

    n_real = len(seqs)
    n_seqs = max(n_real, pad_seqs_to) if decode else n_real
    n_tokens = sum(len(s.tokens) for s in seqs) + (n_seqs - n_real)
    n_want_real = sum(len(s.want) for s in seqs)
    n_want = n_want_real + (n_seqs - n_real if pad_seqs_to else 0)   # a padded step also wants its padding rows
    kv_lens = [b + len(s.tokens) for b, s in zip(bases, seqs)]
    max_kv = max(kv_lens)

    # layout of the block
    off = {}
    cur = 0
    for name, n in (("token_ids", n_tokens), ("tok_seq", n_tokens), ("tok_pos", n_tokens), ("want_rows", max(n_want, 1)),
                    ("seq_q_start", n_seqs + 1), ("seq_kv_len", n_seqs), ("seq_slot", n_seqs)):
        off[name] = (cur, n)
        cur = _align(cur + n)
    page_layout = []
    for g in cache.kv_groups:
        P = max(pages_for(max_kv, g.page_size), pad_pages_to, 1)
        page_layout.append((g, cur, P))
        cur = _align(cur + n_seqs * P)
    host, dev = buffers.stage(cur)
    h = host.numpy()

    tok = h[off["token_ids"][0]:off["token_ids"][0] + n_tokens]
    tseq = h[off["tok_seq"][0]:off["tok_seq"][0] + n_tokens]
    tpos = h[off["tok_pos"][0]:off["tok_pos"][0] + n_tokens]
    want = h[off["want_rows"][0]:off["want_rows"][0] + max(n_want, 1)]
    qstart = h[off["seq_q_start"][0]:off["seq_q_start"][0] + n_seqs + 1]
    kvlen = h[off["seq_kv_len"][0]:off["seq_kv_len"][0] + n_seqs]
    sslot = h[off["seq_slot"][0]:off["seq_slot"][0] + n_seqs]
    t = 0
    w = 0
    want[:] = 0
    for i, (s, base) in enumerate(zip(seqs, bases)):
        n = len(s.tokens)
        tok[t:t + n] = np.asarray(s.tokens, dtype=np.int32)
        tseq[t:t + n] = i
        tpos[t:t + n] = np.arange(base, base + n, dtype=np.int32)
        qstart[i] = t
        kvlen[i] = base + n
        sslot[i] = s.slot
        for place in s.want:
            want[w] = t + int(place)
            w += 1
        t += n
    for i in range(n_real, n_seqs):        # padding sequences: one token that no kernel touches
        tok[t] = -1
        tseq[t] = -1
        tpos[t] = 0
        qstart[i] = t
        kvlen[i] = 0
        sslot[i] = -1
        if pad_seqs_to:
            want[w] = t
            w += 1
        t += 1
    qstart[n_seqs] = t
    for g, start, P in page_layout:
        table = h[start:start + n_seqs * P].reshape(n_seqs, P)
        table[:] = -1
        for i, s in enumerate(seqs):
            pages = g.pool.table(s.slot)
            table[i, :len(pages)] = pages
    buffers.upload(cur)

    ctx = StepContext()
    ctx.n_tokens, ctx.n_seqs, ctx.n_want = n_tokens, n_seqs, n_want
    ctx.n_want_real = n_want_real
    ctx.n_real_seqs = n_real
    ctx.max_q_len = max(len(s.tokens) for s in seqs)
    ctx.max_kv_len = max_kv
    ctx.decode = decode
    ctx.n_q_blocks = sum((len(s.tokens) + 127) // 128 for s in seqs)     # 128-query blocks of the prompt kernel
    ctx.h2d_bytes = cur * 4

    def view(name):
        a, n = off[name]
        return dev[a:a + n]
    ctx.token_ids, ctx.tok_seq, ctx.tok_pos = view("token_ids"), view("tok_seq"), view("tok_pos")
    ctx.want_rows = view("want_rows")[:n_want] if n_want else None
    ctx.seq_q_start, ctx.seq_kv_len, ctx.seq_slot = view("seq_q_start"), view("seq_kv_len"), view("seq_slot")
    for g, start, P in page_layout:
        ctx._pages[id(g)] = dev[start:start + n_seqs * P].view(n_seqs, P)
    return ctx
