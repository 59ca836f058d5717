"""A step's batch: validation on the host, and the index arrays the kernels read.

One step runs the next tokens of some sequences: any number of tokens each, at any
cache length — prompts of unequal lengths that start together, one token each (decode),
or a prompt that goes on in portions beside sequences that decode, as the reference's
``forward_cached`` takes T >= 1 new tokens at any length (include/llmi/model/transformer.hpp:89-95;
used for a chat's next turn, apps/llmi-chat/main.cpp:137-146).  The reference's step takes
one sequence (src/model/transformer.cpp:192-212); its checks are kept per sequence: no
tokens, id out of range, cache full, context exceeded — plus a slot named twice.  A step
whose sequences all bring one token runs the decode kernels; every other step runs the
prompt kernels, which take a sequence's earlier positions from the cache.  Tokens are flattened in sequence order; each token carries the index of its
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

    Two host blocks alternate, each guarded by a mark behind its copy, so that writing the next step's
    arrays never overtakes a copy that is still queued on the stream.
    """

    def __init__(self, device, rt=None):
        self.device = device
        self.rt = rt
        self.hosts = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.dev = None
        self.serial = 0          # counts staged blocks: tells whether anyone used the buffers in between

    def stage(self, n_int32: int):
        """-> (host block to fill, device block); call ``upload`` when the host block is filled."""
        self.turn ^= 1
        self.serial += 1
        i = self.turn
        if self.events[i] is not None:
            self.events[i].wait()
        if self.hosts[i] is None or self.hosts[i].numel() < n_int32:
            self.hosts[i] = torch.empty(max(4096, 2 * n_int32), dtype=torch.int32, pin_memory=True)
        if self.dev is None or self.dev.numel() < n_int32:
            self.dev = torch.empty(max(4096, 2 * n_int32), dtype=torch.int32, device=self.device)
            if self.rt is not None:
                self.rt.generation += 1
        return self.hosts[i], self.dev

    def upload(self, n_int32: int) -> None:
        from ..ops import kernels
        i = self.turn
        if self.events[i] is None:
            self.events[i] = kernels.Mark()
        kernels.copy_to_device(self.dev.data_ptr(), self.hosts[i].data_ptr(), 4 * n_int32, self.events[i])


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
              pad_pages_to: int = 0, pad_tokens_to: int = 0, pad_want_to: int = 0) -> StepContext:
    """Validate a step, reserve its cache room, and upload its index arrays.

    ``pad_seqs_to`` / ``pad_pages_to`` round the decode batch and the page tables up (padding
    sequences have index -1 and are skipped by every kernel) so that recorded launches of one
    shape can be replayed for smaller batches.  ``pad_tokens_to`` (with ``pad_want_to``) does the same
    for a prompt step: token rows up to that number belong to no sequence (id and sequence -1: the
    embedding leaves zeros there and nothing of them reaches the cache or another row), padding
    sequences bring no tokens, and wanted rows beyond the real ones point nowhere (-1).
    """
    if not seqs:
        raise StepError("step: no sequences")
    cache.settle()                 # positions reserved ahead of a step that did not come go back first
    n_real = len(seqs)
    lens = [len(s.tokens) for s in seqs]
    if min(lens) == 0:
        raise StepError("step: a sequence brings no tokens")
    slots = [s.slot for s in seqs]
    if len(set(slots)) != n_real:
        dup = next(x for x in slots if slots.count(x) > 1)
        raise StepError(f"step: slot {dup} is named twice")
    decode = max(lens) == 1
    if decode:
        all_tokens = np.fromiter((s.tokens[0] for s in seqs), dtype=np.int64, count=n_real)
    else:
        all_tokens = np.concatenate([np.asarray(s.tokens, dtype=np.int64) for s in seqs])
    if all_tokens.min() < 0 or all_tokens.max() >= vocab_size:
        bad = int(all_tokens[(all_tokens < 0) | (all_tokens >= vocab_size)][0])
        raise StepError(f"step: token id {bad} out of range")
    for s, n in zip(seqs, lens):
        for w in s.want:
            if not (0 <= int(w) < n):
                raise StepError(f"step: wanted place {w} is not among the {n} tokens given")
    bases = [cache.length(slot) for slot in slots]          # raises CacheError for a slot that is not live
    cache.extend_all(dict(zip(slots, lens)))       # raises with nothing reserved if the step does not fit (it first takes back what was reserved ahead)

    pad_prompt = (not decode) and pad_tokens_to > 0
    n_seqs = max(n_real, pad_seqs_to) if (decode or pad_prompt) else n_real
    n_pad = n_seqs - n_real
    n_want_real = sum(len(s.want) for s in seqs)
    if decode:
        n_tokens = sum(lens) + n_pad
        n_want = n_want_real + (n_pad if pad_seqs_to else 0)   # a padded step also wants its padding rows
    else:
        n_tokens = max(sum(lens), pad_tokens_to)
        n_want = max(n_want_real, pad_want_to) if pad_prompt else n_want_real
    kv_lens = [b + n for b, n in zip(bases, lens)]
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

    def region(name):
        a, n = off[name]
        return h[a:a + n]
    tok, tseq, tpos = region("token_ids"), region("tok_seq"), region("tok_pos")
    want, qstart, kvlen, sslot = region("want_rows"), region("seq_q_start"), region("seq_kv_len"), region("seq_slot")
    n_tok_real = sum(lens)
    tok[:n_tok_real] = all_tokens
    if decode:
        tseq[:n_real] = np.arange(n_real, dtype=np.int32)
        tpos[:n_real] = bases
        qstart[:n_real] = np.arange(n_real, dtype=np.int32)
    else:
        starts = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        tseq[:n_tok_real] = np.repeat(np.arange(n_real, dtype=np.int32), lens)
        tpos[:n_tok_real] = np.arange(n_tok_real, dtype=np.int32) - np.repeat(starts[:-1], lens) + np.repeat(
            np.asarray(bases, dtype=np.int32), lens)
        qstart[:n_real] = starts[:-1]
    kvlen[:n_real] = kv_lens
    sslot[:n_real] = slots
    want[:] = 0
    w = 0
    for i, s in enumerate(seqs):
        for place in s.want:
            want[w] = qstart[i] + int(place)
            w += 1
    if not decode and (n_tokens > n_tok_real or n_pad or n_want > n_want_real):
        # a padded prompt step: rows of no sequence, sequences of no tokens, wanted rows that point nowhere
        tok[n_tok_real:] = -1
        tseq[n_tok_real:] = -1
        tpos[n_tok_real:] = 0
        qstart[n_real:n_seqs] = n_tok_real
        kvlen[n_real:] = 0
        sslot[n_real:] = -1
        want[w:] = -1
    if decode and n_pad:                    # padding sequences: one token each that no kernel touches
        t0 = n_tok_real
        tok[t0:] = -1
        tseq[t0:] = -1
        tpos[t0:] = 0
        qstart[n_real:n_seqs] = np.arange(t0, t0 + n_pad, dtype=np.int32)
        kvlen[n_real:] = 0
        sslot[n_real:] = -1
        if pad_seqs_to:
            want[w:w + n_pad] = np.arange(t0, t0 + n_pad, dtype=np.int32)
    qstart[n_seqs] = n_tokens if decode else n_tok_real
    slot_index = np.asarray(slots, dtype=np.int64)
    for g, start, P in page_layout:
        table = h[start:start + n_seqs * P].reshape(n_seqs, P)
        m = g.pool.matrix
        if m is not None and P <= m.shape[1] and slot_index.max() < m.shape[0]:
            table[:n_real] = m[slot_index, :P]
            table[n_real:] = -1
        else:
            table[:] = -1
            for i, slot in enumerate(slots):
                pages = g.pool.table(slot)
                table[i, :len(pages)] = pages
    buffers.upload(cur)

    ctx = StepContext()
    ctx.n_tokens, ctx.n_seqs, ctx.n_want = n_tokens, n_seqs, n_want
    ctx.n_want_real = n_want_real
    ctx.n_real_seqs = n_real
    ctx.max_q_len = max(lens)
    ctx.max_kv_len = max_kv
    ctx.decode = decode
    # 128-query blocks of the prompt kernel; a padded step launches the most that its shape can have (the rest find no work)
    ctx.n_q_blocks = (n_tokens // 128 + n_seqs) if pad_prompt else sum((n + 127) // 128 for n in lens)
    # for kernels that plan on the host (a padded step's launches must not depend on its lengths)
    ctx.host_q_lens, ctx.host_kv_lens = (None, None) if (decode or pad_prompt) else (list(lens), list(kv_lens))
    ctx.h2d_bytes = cur * 4

    def view(name):
        a, n = off[name]
        return dev[a:a + n]
    ctx.token_ids, ctx.tok_seq, ctx.tok_pos = view("token_ids"), view("tok_seq"), view("tok_pos")
    ctx.want_rows = view("want_rows")[:n_want] if n_want else None
    ctx.seq_q_start, ctx.seq_kv_len, ctx.seq_slot = view("seq_q_start"), view("seq_kv_len"), view("seq_slot")
    for g, start, P in page_layout:
        ctx._pages[id(g)] = dev[start:start + n_seqs * P].view(n_seqs, P)
    ctx.layout = StepLayout(off, page_layout, cur, host, tuple(slots))
    return ctx


@dataclass
class StepLayout:
    """Where a step's arrays lie in its index block, and the host block that holds them."""
    offsets: dict            # name -> (start, count)
    pages: list              # (group, start, pages per sequence)
    n_int32: int
    host: torch.Tensor
    slots: tuple


def continue_decode_step(cache, prev: StepContext, tokens, vocab_size: int, buffers: StepBuffers) -> None:
    """The index block of a decode step that continues ``prev`` (a decode step of the same slots, padded to
    the same sizes) by one token each: only the token ids, the positions, the lengths and the page tables
    change, so the block is copied and patched instead of being planned anew.  The checks are those of
    :func:`plan_step`.  The caller makes sure that the page tables still fit ``prev``'s width."""
    toks = _check_continuing_tokens(prev, tokens, vocab_size)
    bases = cache.extend_each_by_one(prev.layout.slots)
    host = _patched_block(prev, bases, buffers)
    _finish_block(prev, host, toks, bases, buffers)


@dataclass
class PendingStep:
    """A continued decode step laid out ahead of its tokens (see :func:`prepare_continue`)."""
    host: torch.Tensor
    bases: "np.ndarray"
    serial: int


def prepare_continue(cache, prev: StepContext, buffers: StepBuffers) -> PendingStep:
    """Everything of :func:`continue_decode_step` that does not need the tokens, done while the device still runs
    ``prev``: the next positions are reserved ahead (``cache.speculate_each_by_one``) and the block is copied and
    patched.  :func:`finish_continue` adds the tokens and uploads it; if the step never comes, ``cache.settle()``
    takes the reservation back and the block is forgotten.  Raises CacheError (nothing reserved) if the cache has
    no room or cannot reserve ahead."""
    bases = cache.speculate_each_by_one(prev.layout.slots)
    host = _patched_block(prev, bases, buffers)
    return PendingStep(host, bases, buffers.serial)


def finish_continue(cache, prev: StepContext, pending: PendingStep, tokens, vocab_size: int, buffers: StepBuffers) -> None:
    """The tokens of a step laid out by :func:`prepare_continue` have come: check them, upload the block, and let
    the reserved positions count.  A bad token id raises with the reservation taken back."""
    try:
        toks = _check_continuing_tokens(prev, tokens, vocab_size)
    except StepError:
        cache.settle()
        raise
    cache.commit_speculation()
    _finish_block(prev, pending.host, toks, pending.bases, buffers)


def _check_continuing_tokens(prev: StepContext, tokens, vocab_size: int):
    n_real = len(prev.layout.slots)
    toks = np.asarray(tokens, dtype=np.int64)
    if toks.shape != (n_real,):
        raise StepError("step: one token for each sequence of the step before")
    if toks.min() < 0 or toks.max() >= vocab_size:
        bad = int(toks[(toks < 0) | (toks >= vocab_size)][0])
        raise StepError(f"step: token id {bad} out of range")
    return toks


def _patched_block(prev: StepContext, bases, buffers: StepBuffers):
    """A fresh host block holding ``prev``'s arrays with positions, lengths and page tables one token on."""
    lay = prev.layout
    n_real = len(lay.slots)
    host, _ = buffers.stage(lay.n_int32)
    h = host.numpy()
    h[:lay.n_int32] = lay.host.numpy()[:lay.n_int32]
    a = lay.offsets["tok_pos"][0]
    h[a:a + n_real] = bases
    a = lay.offsets["seq_kv_len"][0]
    h[a:a + n_real] = bases + 1
    slot_index = np.asarray(lay.slots, dtype=np.int64)
    n_seqs = prev.n_seqs
    for g, start, P in lay.pages:
        table = h[start:start + n_seqs * P].reshape(n_seqs, P)
        m = g.pool.matrix
        if m is not None and P <= m.shape[1] and slot_index.max() < m.shape[0]:
            table[:n_real] = m[slot_index, :P]
        else:
            table[:n_real] = -1
            for i, slot in enumerate(lay.slots):
                pages = g.pool.table(slot)
                table[i, :len(pages)] = pages
    return host


def _finish_block(prev: StepContext, host, toks, bases, buffers: StepBuffers) -> None:
    lay = prev.layout
    a = lay.offsets["token_ids"][0]
    host.numpy()[a:a + len(lay.slots)] = toks
    buffers.upload(lay.n_int32)
    lay.host = host
    prev.max_kv_len = int(bases.max()) + 1
