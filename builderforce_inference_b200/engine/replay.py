"""Trace replay: feeds given token ids through a model step by step and writes logits.

    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps arrive on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry brings the next tokens of one request and the places among them whose logits are
wanted.  For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits at
the wanted places, in the order of the entries and of ``want``, as little-endian float32
``[wanted, vocab]``.  After every step a line ``done <step>`` is printed and flushed.  Requests
named in ``end`` give back what they hold after the step.  Nothing is sampled.

There is no model code here: the loop drives the package's engine (model, step function, cache,
kernels), the same one generation uses.  ``bin/trace_run`` and the command line's ``replay``
subcommand both run this function.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def add_arguments(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")


def replay(args, lines=None) -> int:
    print("trace_run: loading the engine (kernels are compiled on first use)", file=sys.stderr, flush=True)
    import torch

    from .engine import Engine, SequenceStep

    os.makedirs(args.out, exist_ok=True)
    engine = Engine.load(args.model, dtype=args.dtype, max_tokens=args.max_tokens, device=args.device)
    slots = {}
    for line in (sys.stdin if lines is None else lines):
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        seqs = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slots:
                slots[rid] = engine.acquire()
            seqs.append(SequenceStep(slot=slots[rid], tokens=e["tokens"], want=e.get("want", [])))
        if seqs:
            logits = engine.step(seqs)
            if logits.shape[0] > 0:
                host = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                with open(tmp, "wb") as f:
                    f.write(host.tobytes())
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
            else:
                torch.cuda.synchronize()
        for rid in rec.get("end", []):
            if rid in slots:
                engine.release(slots.pop(rid))
        print(f"done {step}", flush=True)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="replay a token trace through the engine and write logits")
    add_arguments(ap)
    return replay(ap.parse_args(argv))
