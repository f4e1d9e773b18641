"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives the same model,
step function, cache and kernels that generation uses.  The reference's nearest tool feeds a
text's tokens one by one through its forward and can save per-position rows
(tools/quant.c:430-720, --ppl with --save-logits).

Input (standard input), one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits at the wanted
places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import torch
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    from . import Engine, StepEntry, load_model

    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, args.device)
    engine = Engine(model, max_tokens=args.max_tokens, device=args.device)
    live: Dict[str, object] = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in live:
                live[rid] = engine.open()
            entries.append(StepEntry(live[rid], e["tokens"], e.get("want", [])))
        logits = engine.step(entries)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            engine.check_kernels()          # a tensor-core kernel that gave up on a wait must not pass for a result
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            seq = live.pop(str(rid), None)
            if seq is not None:
                engine.close(seq)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
