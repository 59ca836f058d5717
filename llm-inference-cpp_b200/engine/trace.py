"""Trace replay: feed given token ids through the model step by step and write the logits.

The reference's counterpart is ``llmi-generate --dump`` driven by a script
(apps/llmi-generate/main.cpp:85-97, 300-313; tools/crosscheck_forward.py:116-119): one
whole-sequence pass whose states and logits go to a file.  This replay goes through the
cache instead: every step brings each request's next tokens, and the logits of the wanted
places are written as little-endian fp32 ``[wanted, vocab]``.  It samples nothing, and it has
no forward pass, cache or loader of its own: it calls the model's ``step`` on the model's
cache, the same ones generation uses.
"""
from __future__ import annotations

import json
import os
import sys

from ..cache.pages import PAGE_SIZE
from .batch import SequenceStep
from .loader import load_model


class TraceReplayer:
    def __init__(self, model, max_tokens: int):
        self.model = model
        self.cache = model.new_cache(max(max_tokens, PAGE_SIZE))
        self.slots: dict[str, int] = {}

    def run_step(self, step: dict):
        """One line of the trace.  Returns fp32 logits [wanted, vocab] on the host, or None."""
        entries = step.get("entries", [])
        seqs = []
        for e in entries:
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = self.cache.alloc_slot()
            seqs.append(SequenceStep(self.slots[rid], [int(t) for t in e["tokens"]], [int(w) for w in e.get("want", [])]))
        logits = None
        if seqs:
            out = self.model.step(self.cache, seqs)
            if out.shape[0] > 0:
                logits = out.cpu().numpy()
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.cache.free_slot(self.slots.pop(rid))
        return logits


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids through the model and write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help=f"most tokens live requests hold at once (each rounded up to {PAGE_SIZE})")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, args.device)
    replayer = TraceReplayer(model, args.max_tokens)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        logits = replayer.run_step(step)
        if logits is not None:
            logits.astype("<f4").tofile(os.path.join(args.out, f"{step['step']}.f32"))
        print(f"done {step['step']}", flush=True)
    return 0
