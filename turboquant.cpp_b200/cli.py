"""Command line in the manner of the reference's `quant` tool (tools/quant.c:126-163, 241-346).

    quant <model folder> | --random CONFIG.json [--seed-weights N]
          [-p "ids"]… [--tokens-file FILE] [-n max_tokens] [-T temperature] [-P top_p] [-s seed]
          [--ctx N] [--dtype bfloat16|float32] [--batch N] [--stop id]… [--rep-penalty F] [--rep-window N]
          [--detect-loops] [--info] [--profile]
          [--bench-prefill] [--bench-memory]

Names and meanings follow the reference where it has them: -p prompt (default "Hello" there; here
a prompt is a list of token ids, "1,2,3" or "1 2 3", default "0"), -n max tokens (256), -T
temperature (0.7), -P top-p (0.9), -s seed (42; 0 means the default), --ctx context length, --info
print the model and exit, --profile the share and time per token of matmul / moe / attn / other as the reference
prints them (src/engine/tq_transformer.c:2994-3021) plus each bucket's bytes and operations against the device's
peaks, --bench-prefill and --bench-memory (decode speed at growing context).  Instead of a model folder,
--random CONFIG.json runs the configuration with random weights drawn from --seed-weights (the reference has
no such mode; its tests fill weights by hand).  --tokens-file FILE reads prompts from a file, one per line
(the reference reads its text prompts from a file the same way for --ppl, tools/quant.c:430-470).
TQ_DEBUG_LAYERS=1 in the environment prints per-layer checksums of the residual stream as the reference's
TQ_DEBUG_PREFILL does.  --rep-penalty and --rep-window set what the reference keeps as
engine defaults without an option (1.1 over 32 tokens, include/turboquant/tq_engine.h:408-409); here
the penalty is off unless asked for, and so is the reference's detector of repetition loops
(--detect-loops; src/engine/tq_generate.c:610-630).  -j (threads) is accepted and ignored.  -p may be given several
times: the prompts run as batches.  Token ids go to stdout, one line per prompt; the summary
"N tokens in X s (Y tok/s)" goes to stderr as the reference prints it (tools/quant.c:1371-1376).
"""
from __future__ import annotations

import argparse
import sys
import time
from typing import List


def parse_ids(text: str) -> List[int]:
    parts = text.replace(",", " ").split()
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit(f"quant: a prompt is a list of token ids (\"1,2,3\"), got {text!r}") from None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="quant", description="Generate tokens with a model folder on one B200.")
    ap.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG.json", help="a configuration to run with random weights instead of a folder")
    ap.add_argument("--seed-weights", type=int, default=0, help="seed of the random weights (with --random)")
    ap.add_argument("-p", dest="prompts", action="append", help="prompt as token ids; may repeat")
    ap.add_argument("--tokens-file", help="file with one prompt (token ids) per line; empty lines and # lines are skipped")
    ap.add_argument("-n", dest="max_tokens", type=int, default=256)
    ap.add_argument("-T", dest="temperature", type=float, default=0.7)
    ap.add_argument("-P", dest="top_p", type=float, default=0.9)
    ap.add_argument("-s", dest="seed", type=int, default=42)
    ap.add_argument("-j", dest="threads", type=int, default=0, help="accepted for compatibility; ignored")
    ap.add_argument("--ctx", type=int, default=0, help="context length per request (default: model's, at most 4096)")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--batch", type=int, default=8, help="most requests in one batch")
    ap.add_argument("--stop", type=int, action="append", help="stop token id; may repeat (default: the model's eos)")
    ap.add_argument("--rep-penalty", type=float, default=1.0,
                    help="repetition penalty over the last --rep-window tokens (the reference's engine applies 1.1; 1 = off)")
    ap.add_argument("--rep-window", type=int, default=32)
    ap.add_argument("--detect-loops", action="store_true",
                    help="end a request whose last four tokens have come up three times before (the reference always does)")
    ap.add_argument("--info", action="store_true")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--bench-prefill", action="store_true")
    ap.add_argument("--bench-memory", action="store_true")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    import json
    import os
    from .config.registry import load_config, parse_config
    from . import models  # noqa: F401
    if (args.model is None) == (args.random is None):
        ap.error("give a model folder or --random CONFIG.json (one of the two)")
    raw = None
    if args.random is not None:
        try:
            with open(args.random, encoding="utf-8") as f:
                raw = json.load(f)
        except (OSError, ValueError) as e:
            print(f"quant: cannot read the configuration '{args.random}': {e}", file=sys.stderr)
            return 2
    if args.profile:
        os.environ.setdefault("TQ_NO_PDL", "1")       # a kernel's time without its wait for the one before
        os.environ.setdefault("TQ_NO_GRAPHS", "1")    # kernels launched one by one show up under their names
    if args.info:
        arch, cfg = parse_config(raw, args.random) if raw is not None else load_config(args.model)
        print(f"architecture: {arch.name}")
        for k, v in sorted(cfg.to_dict().items()):
            print(f"  {k}: {v}")
        return 0

    import torch
    if not torch.cuda.is_available():
        print("quant: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    from .model import Model
    seed = args.seed if args.seed != 0 else 42
    options = dict(temperature=args.temperature, top_p=args.top_p, max_tokens=args.max_tokens,
                   context_length=args.ctx, seed=seed, device=args.device, max_batch=args.batch,
                   stop_token_ids=args.stop, rep_penalty=args.rep_penalty, rep_window=args.rep_window,
                   detect_loops=args.detect_loops)
    if raw is not None:
        from .engine.loading import random_model
        m = Model.from_model(random_model(raw, args.seed_weights, args.dtype, args.device), **options)
    else:
        m = Model(args.model, dtype=args.dtype, **options)
    if args.bench_prefill or args.bench_memory:
        from .engine.bench_tools import bench_memory, bench_prefill
        if args.bench_prefill:
            bench_prefill(m, file=sys.stderr)
        if args.bench_memory:
            bench_memory(m, file=sys.stderr)
        return 0
    prompts = [parse_ids(p) for p in (args.prompts or [])]
    if args.tokens_file:
        try:
            with open(args.tokens_file, encoding="utf-8") as f:
                prompts += [parse_ids(line) for line in f if line.strip() and not line.lstrip().startswith("#")]
        except OSError as e:
            print(f"quant: cannot read the prompts' file '{args.tokens_file}': {e}", file=sys.stderr)
            return 2
    if not prompts:
        prompts = [parse_ids("0")]
    t0 = time.perf_counter()
    if args.profile:
        from .engine.bench_tools import device_peaks, profile_generation
        hbm, tf = device_peaks()
        outs = profile_generation(m, prompts, hbm, tf, file=sys.stderr)["outs"]
    else:
        outs = m.generate_batch(prompts)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for o in outs:
        print(" ".join(str(t) for t in o))
    n = sum(len(o) for o in outs)
    st = m.last_stats
    print(f"{n} tokens in {dt:.2f} s ({n / dt:.1f} tok/s; prefill {st.prompt_tokens} tokens in "
          f"{st.prefill_seconds:.3f} s, decode {st.decode_seconds:.3f} s, {st.batches} batches)", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
