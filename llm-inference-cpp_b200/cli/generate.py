"""``llmi-generate``: generation from a model folder, in the manner of the reference's command line.

Option names and meanings are the reference's where it has them
(apps/llmi-generate/main.cpp:205-264; ``--top-k`` from apps/llmi-chat/main.cpp:44-59):

    llmi-generate MODEL_DIR --ids N,N,... [--max-new N] [--ignore-eos] [--json] [--dump FILE]
                  [--kv-cache] [--temperature T] [--top-k N] [--top-p P] [--seed N]
                  [--dtype bf16|fp32] [--ids-file FILE] [--max-batch N]
    llmi-generate --random CONFIG.json [--seed-weights S] --ids ...

``--max-new`` defaults to 32; generation is greedy unless ``--temperature`` is given; stop
tokens are the configuration's ``eos_token_id`` unless ``--ignore-eos``.  ``--json`` prints
``prompt_ids``, ``generated_ids``, ``load_seconds``, ``generate_seconds`` and ``weight_bytes``
(main.cpp:339-344).  ``--dump FILE`` writes one whole-prompt pass as the reference does
(main.cpp:85-97): a JSON header line, then fp32 little-endian states and all-position logits.
``--kv-cache`` is accepted and changes nothing: this engine always runs from its cache.
``--ids-file`` holds one comma-separated prompt per line; the prompts run as batches.
Text prompts need a tokenizer, which this library does not have: ``--prompt`` is refused.
Exit codes: 2 for a usage error, 1 for a runtime error (main.cpp:206-211, 268-276).
"""
from __future__ import annotations

import json
import sys
import time

USAGE = ("usage: llmi-generate (MODEL_DIR | --random CONFIG.json [--seed-weights S]) (--ids N,N,... | --ids-file FILE) "
         "[--max-new N] [--ignore-eos] [--json] [--dump FILE] [--kv-cache] [--temperature T] [--top-k N] [--top-p P] "
         "[--seed N] [--dtype bf16|fp32] [--max-batch N]\n")


def parse_ids(s: str):
    """Comma-separated non-negative integers of at most nine digits (main.cpp:53-64); None if malformed."""
    out = []
    for part in s.split(","):
        if not part or not part.isdigit() or not part.isascii() or len(part) > 9:
            return None
        out.append(int(part))
    return out or None


class UsageError(Exception):
    pass


def parse_args(argv):
    if len(argv) < 1:
        raise UsageError(USAGE.rstrip())
    opts = {"dir": None, "random": None, "seed_weights": 0, "ids": [], "max_new": 32, "ignore_eos": False, "json": False,
            "dump": None, "temperature": 0.0, "top_k": 0, "top_p": 1.0, "seed": 0, "dtype": "bf16", "max_batch": 64,
            "prompt": None}
    i = 0
    if not argv[0].startswith("--"):
        opts["dir"] = argv[0]
        i = 1
    valued = {"--ids", "--ids-file", "--max-new", "--dump", "--temperature", "--top-k", "--top-p", "--seed", "--dtype",
              "--random", "--seed-weights", "--max-batch", "--prompt", "--quant"}
    while i < len(argv):
        a = argv[i]
        if a in valued and i + 1 < len(argv):
            v = argv[i + 1]
            i += 2
            try:
                if a == "--ids":
                    ids = parse_ids(v)
                    if ids is None:
                        raise UsageError("error: --ids takes comma-separated token ids")
                    opts["ids"].append(ids)
                elif a == "--ids-file":
                    with open(v) as f:
                        for line in f:
                            if line.strip():
                                ids = parse_ids(line.strip())
                                if ids is None:
                                    raise UsageError("error: --ids-file takes one comma-separated prompt per line")
                                opts["ids"].append(ids)
                elif a == "--max-new":
                    opts["max_new"] = int(v)
                elif a == "--dump":
                    opts["dump"] = v
                elif a == "--temperature":
                    opts["temperature"] = float(v)
                elif a == "--top-k":
                    opts["top_k"] = int(v)
                elif a == "--top-p":
                    opts["top_p"] = float(v)
                elif a == "--seed":
                    opts["seed"] = int(v)
                elif a == "--dtype":
                    opts["dtype"] = v
                elif a == "--random":
                    opts["random"] = v
                elif a == "--seed-weights":
                    opts["seed_weights"] = int(v)
                elif a == "--max-batch":
                    opts["max_batch"] = int(v)
                elif a == "--prompt":
                    opts["prompt"] = v
                elif a == "--quant":
                    if v != "f32":
                        raise UsageError("error: quantized weights are not part of this library; --quant takes f32 only")
            except (ValueError, OSError) as e:
                raise UsageError(f"error: bad value for {a}: {e}") from None
        elif a == "--ignore-eos":
            opts["ignore_eos"] = True
            i += 1
        elif a == "--json":
            opts["json"] = True
            i += 1
        elif a == "--kv-cache":
            i += 1
        else:
            raise UsageError(f"error: unknown or incomplete argument {a}")
    if opts["dir"] is None and opts["random"] is None:
        raise UsageError(USAGE.rstrip())
    return opts


def write_dump(path, states, logits, tokens, hidden, vocab):
    import numpy as np
    with open(path, "wb") as f:
        f.write((json.dumps({"tokens": tokens, "hidden": hidden, "vocab": vocab, "states": len(states)},
                            separators=(",", ":")) + "\n").encode())
        for s in states:
            f.write(np.ascontiguousarray(s, dtype="<f4").tobytes())
        f.write(np.ascontiguousarray(logits, dtype="<f4").tobytes())


def run(argv) -> int:
    try:
        o = parse_args(argv)
    except UsageError as e:
        sys.stderr.write(str(e) + "\n")
        return 2
    if o["prompt"] is not None:
        sys.stderr.write("error: this library has no tokenizer; pass --ids instead\n")
        return 1
    if not o["ids"]:
        sys.stderr.write("error: give --prompt or --ids\n")
        return 2

    from .. import SamplingParams, SequenceStep, generate, load_model, random_model
    t0 = time.perf_counter()
    try:
        if o["random"] is not None:
            with open(o["random"]) as f:
                model = random_model(json.load(f), o["seed_weights"], o["dtype"])
        else:
            model = load_model(o["dir"], o["dtype"])
    except Exception as e:  # every loader error is reported the same way, as the reference does
        sys.stderr.write(f"error: {e}\n")
        return 1
    load_s = time.perf_counter() - t0

    try:
        if o["dump"]:
            ids = o["ids"][0]
            cache = model.new_cache(max(64, (len(ids) + 63) // 64 * 64))
            slot = cache.alloc_slot()
            states = []
            logits = model.step(cache, [SequenceStep(slot, ids, list(range(len(ids))))], trace=states).cpu().numpy()
            cache.free_slot(slot)
            write_dump(o["dump"], [s.cpu().numpy() for s in states], logits, len(ids), model.spec.width, model.vocab_size)
            if o["max_new"] == 0:
                return 0
        t1 = time.perf_counter()
        sampling = SamplingParams(o["temperature"], o["top_k"], o["top_p"], o["seed"])
        outs = generate(model, o["ids"], max_new=o["max_new"], ignore_eos=o["ignore_eos"], sampling=sampling,
                        max_batch=o["max_batch"])
        gen_s = time.perf_counter() - t1
    except Exception as e:
        sys.stderr.write(f"error: {e}\n")
        return 1

    if o["json"]:
        for ids, out in zip(o["ids"], outs):
            print(json.dumps({"prompt_ids": ids, "generated_ids": out, "load_seconds": round(load_s, 3),
                              "generate_seconds": round(gen_s, 3), "weight_bytes": model.weight_bytes()},
                             separators=(",", ":")))
        return 0
    for out in outs:
        print("generated ids: " + ",".join(map(str, out)))
    n_prompt = sum(len(p) for p in o["ids"])
    n_out = sum(len(x) for x in outs)
    print(f"[{n_prompt} prompt tokens, {n_out} generated in {gen_s:.2f} s ({n_out / max(gen_s, 1e-9):.2f} tokens/s, "
          f"KV cache); load {load_s:.2f} s; {model.weight_bytes()} weight bytes]")
    return 0


def main() -> int:
    try:
        return run(sys.argv[1:])
    except Exception as e:
        sys.stderr.write(f"error: {e}\n")
        return 1
