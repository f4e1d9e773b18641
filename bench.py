#!/usr/bin/env python3
"""Decode and prefill speed of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model a2.7b|57b] [--layers L] [--batch B]
                    [--impl reference]

The model has the layer sizes of Qwen1.5-MoE-A2.7B (default) or of Qwen2-57B-A14B (--model 57b) with seeded
random weights in bfloat16; token ids are synthetic (uniform).  A "step" is one decode step of a batch of 8
sequences that start from 2,048-token prompts (cache for 4,096 each).  One JSON line is printed:
  value     decoded tokens per second, timed on the device with CUDA events over exactly K steps
            (every step reads far more weight and cache bytes than the L2 holds, so no flush)
  e2e       the same through the Python entry point (Model.generate_batch): host token ids in,
            host token ids out, every step's host-to-device and device-to-host copies included
  prefill   one 2,048-token prompt: tokens per second, milliseconds, fraction of the bf16 peak
  roofline  bytes the decode step has to read (each weight it uses once, and the cache of the live
            requests) / its time, against the measured copy bandwidth
  points    decode tokens per second at batch 1 and batch 64 from 2,048-token prompts, and at batch 1, 8 and 64
            with the context at 4,096 by the last timed step; points_frac: each point's fraction of the roofline
  vs_baseline  against the reference's own CPU forward, timed once on this architecture's sizes (`baseline` says how):
            the reference has no GPU path, no batch and no prompt step for it, so this is context, not a race
Only one GPU is supported: for --gpus N > 1 a line says so and the exit code is 2.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model (Qwen1.5-MoE-A2.7B); weights are random.
A27B = {
    "architectures": ["Qwen2MoeForCausalLM"], "model_type": "qwen2_moe",
    "num_hidden_layers": 24, "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 16,
    "num_experts": 60, "num_experts_per_tok": 4, "moe_intermediate_size": 1408, "norm_topk_prob": False,
    "shared_expert_intermediate_size": 5632, "intermediate_size": 5632, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 8192, "use_sliding_window": False,
    "sliding_window": 0, "max_window_layers": 24, "tie_word_embeddings": False, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "hidden_act": "silu", "torch_dtype": "bfloat16",
}
# Layer sizes of Qwen2-57B-A14B.
B57 = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, num_experts=64,
           num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
           intermediate_size=20480, max_position_embeddings=32768, max_window_layers=28)
MODELS = {"a2.7b": ("Qwen1.5-MoE-A2.7B sizes", A27B), "57b": ("Qwen2-57B-A14B sizes", B57)}
PROMPT, CONTEXT = 2048, 4096


def reference_cpu_rate(layers):
    """Tokens per second of the reference's own CPU forward at Qwen1.5-MoE-A2.7B sizes with `layers` layers, from
    the committed record of one timed run on 1 and 2 layers (tests/golden/reference_cpu_timing.txt, made by
    tests/golden/time_reference.sh): head and embedding once, the layer's cost times the number of layers."""
    try:
        ms = {}
        for line in open(os.path.join(ROOT, "tests", "golden", "reference_cpu_timing.txt")):
            f = line.split()
            if f and f[0] == "layers":
                ms[int(f[1])] = float(f[5])
        layer = ms[2] - ms[1]
        return 1e3 / (ms[1] - layer + layers * layer), ms
    except (OSError, KeyError, ValueError, IndexError):
        return None, {}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            d = json.load(open(p))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)), "source": "measured"}
        except Exception:  # noqa: BLE001 - fall through to the stated fallback
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--id=0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=0)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i].lower() == "active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else 0, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def model_numbers(cfg, layers):
    """Parameter and flop counts from the configuration."""
    H, nh, nkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    E, k, I, S, V = (cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"],
                     cfg["shared_expert_intermediate_size"], cfg["vocab_size"])
    attn = H * (nh + 2 * nkv) * hd + (nh + 2 * nkv) * hd + nh * hd * H
    expert = 3 * H * I
    shared = 3 * H * S + H
    router = E * H
    return dict(attn=attn, expert=expert, shared=shared, router=router, norms=2 * H, head=V * H, embed=V * H,
                layers=layers, kv_per_token=layers * 2 * nkv * hd, H=H, E=E, k=k, V=V, nh=nh, hd=hd)


def decode_bytes(n, distinct_experts_per_layer, batch, context_tokens_total, el=2):
    """Bytes one decode step has to read: every weight it uses once and the live requests' cache."""
    per_layer = n["attn"] + n["shared"] + n["router"] + n["norms"]
    w = n["layers"] * per_layer + sum(distinct_experts_per_layer) * n["expert"] + n["head"] + batch * n["H"] + n["H"]
    return w * el + context_tokens_total * n["kv_per_token"] * el


def prefill_flops(n, T):
    per_tok = 2 * (n["attn"] + n["k"] * n["expert"] + n["shared"] + n["router"])
    attn = 4 * n["nh"] * n["hd"] * T * (T + 1) / 2
    return n["layers"] * (T * per_tok + attn) + 2 * n["head"]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--model", choices=sorted(MODELS), default="a2.7b")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="float32: the true 32-bit path of the whole model (exact kernels, SGEMM without TF32)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points and the prefill")
    ap.add_argument("--kernel-table", default="", help="write a per-kernel time table of a few decode steps and of a "
                    "prefill to this file (torch profiler; not part of any timed number)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C project without setup.py/pyproject.toml at its root (pip install fails), "
                          "and its engine runs this architecture from GGUF on the CPU only: no safetensors MoE, no "
                          "random-weights mode, no CUDA forward"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": f"this library runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.kernels import _call

    pk = peaks()
    model_name, cfg = MODELS[args.model]
    cfg = dict(cfg)
    FULL_LAYERS = cfg["num_hidden_layers"]
    args.layers = args.layers or FULL_LAYERS
    cfg["num_hidden_layers"] = args.layers
    cfg["max_window_layers"] = args.layers
    n = model_numbers(cfg, args.layers)
    torch.cuda.set_device(0)
    t_load = time.time()
    EL = 2 if args.dtype == "bfloat16" else 4                 # bytes per weight and per cached value
    model = tq.random_model(cfg, seed=0, dtype=args.dtype, device="cuda:0")
    torch.cuda.synchronize()
    print(f"[bench] model with {args.layers} layers ready in {time.time() - t_load:.1f} s", file=sys.stderr, flush=True)
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]

    def run_decode(batch, steps, warmup, want_experts=False, prompt=PROMPT):
        """Prefill `batch` prompts of `prompt` tokens, then time `steps` decode steps on the device."""
        eng = tq.Engine(model, max_tokens=batch * CONTEXT, max_slots=batch)
        seqs = [eng.open() for _ in range(batch)]
        group = 8
        for g0 in range(0, batch, group):
            eng.step([tq.StepEntry(s, rng.integers(0, V, size=prompt).tolist(), []) for s in seqs[g0:g0 + group]])
        smp = tq.Sampler(0.0)
        toks = rng.integers(0, V, size=(warmup + steps + 1, batch))

        def one(i):
            logits = eng.step([tq.StepEntry(s, [int(toks[i, j])], [0]) for j, s in enumerate(seqs)])
            return smp.sample(logits, list(range(batch)), [i] * batch)

        distinct = None
        if want_experts:
            eng.debug = {}
            one(0)
            distinct = [int(torch.unique(a).numel()) for a in eng.debug["router_ids"]]
            eng.debug = None
        else:
            one(0)
        for i in range(1, warmup):
            one(i)
        ctx_tokens = sum(s.length for s in seqs)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = _call.LAUNCHES
        torch.cuda.synchronize()
        a.record()
        for i in range(warmup, warmup + steps):
            one(i)
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = _call.LAUNCHES - launches0
        ctx_mid = ctx_tokens + batch * steps // 2
        for s in seqs:
            eng.close(s)
        eng.release()             # the engine's graphs point back at it: without this its cache would stay until a collection
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        return dict(ms_per_step=ms / steps, tok_s=batch * steps / ms * 1e3, launches=launches, distinct=distinct,
                    ctx_tokens=ctx_mid)

    # ---- the headline: decode at the default batch ------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    main_run = run_decode(args.batch, args.steps, args.warmup, want_experts=True)
    clock_rec = clocks.stop()
    dbytes = decode_bytes(n, main_run["distinct"], args.batch, main_run["ctx_tokens"], EL)
    achieved = dbytes / (main_run["ms_per_step"] * 1e-3) / 1e9

    # ---- end to end through the Python entry point ---------------------------------------------------
    m = tq.Model.from_model(model, temperature=0.0, max_tokens=args.steps + 1, context_length=CONTEXT, max_batch=args.batch)
    prompts = [rng.integers(0, V, size=PROMPT).tolist() for _ in range(args.batch)]
    m.generate_batch([p[:64] for p in prompts], max_tokens=4)          # warm-up
    m.generate_batch(prompts)
    st = m.last_stats
    e2e_tok_s = (st.generated_tokens - args.batch) / st.decode_seconds if st.decode_seconds > 0 else 0.0
    h2d = 4 * (7 * args.batch + 1 + args.batch * (CONTEXT // 64))       # packed int32 metadata of a decode step
    d2h = 4 * args.batch
    m.close()

    ref_rate, ref_ms = reference_cpu_rate(args.layers) if args.model == "a2.7b" else (None, {})
    out = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, random weights)", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(main_run["tok_s"] / ref_rate, 1) if ref_rate else None,
        "baseline": ({"value": round(ref_rate, 4), "unit": "tokens/s", "what": "the reference's own forward (tq_forward) on a CPU, "
                      "float32, one token of one sequence at a time: it has no GPU path, no batch and no prompt step for "
                      "this architecture; timed on 1 and 2 layers of these sizes and scaled to this run's layers "
                      "(tests/golden/reference_cpu_timing.txt); other hardware, so context, not a race",
                      "ms_per_token_1_layer": ref_ms.get(1), "ms_per_token_2_layers": ref_ms.get(2)} if ref_rate else None),
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic token ids, seeded random weights", "impl": "ours",
        "config": {"model": model_name, "layers": args.layers, "layers_of_model": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "experts": cfg["num_experts"],
                   "top_k": cfg["num_experts_per_tok"], "moe_inter": cfg["moe_intermediate_size"],
                   "shared_inter": cfg["shared_expert_intermediate_size"], "vocab": V, "global_batch": args.batch,
                   "seq_len": CONTEXT, "prompt_len": PROMPT, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights and cache read per step)"},
        "clocks": clock_rec,
        "e2e": {"value": round(e2e_tok_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": main_run["launches"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"],
                     "bytes_per_step": int(dbytes)},
    }
    if not args.no_points:
        # ---- prefill of one 2,048-token prompt --------------------------------------------------------
        eng = tq.Engine(model, max_tokens=PROMPT, max_slots=1)
        toks = rng.integers(0, V, size=PROMPT).tolist()
        best = float("inf")
        for i in range(4):
            s = eng.open()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            eng.step([tq.StepEntry(s, toks, [PROMPT - 1])])
            b.record()
            torch.cuda.synchronize()
            if i > 0:
                best = min(best, a.elapsed_time(b))
            eng.close(s)
        eng.release()
        del eng
        gc.collect()
        torch.cuda.empty_cache()
        fl = prefill_flops(n, PROMPT)
        out["prefill"] = {"value": round(PROMPT / best * 1e3, 1), "tokens": PROMPT, "ms": round(best, 3),
                          # (no measured peak for float32 products without TF32: no fraction there)
                          "frac": round(fl / (best * 1e-3) / (pk["bf16_tflops"] * 1e12), 4) if EL == 2 else None}
        k_pts = max(8, min(args.steps, 32))
        out["points"], out["points_frac"] = {}, {}
        # from 2,048-token prompts, and with the context at 4,096 by the last timed step
        for name, batch, prompt in (("decode_b1", 1, PROMPT), ("decode_b64", 64, PROMPT),
                                    ("decode_b1_ctx4096", 1, CONTEXT - k_pts - 3), ("decode_b8_ctx4096", 8, CONTEXT - k_pts - 3),
                                    ("decode_b64_ctx4096", 64, CONTEXT - k_pts - 3)):
            r = run_decode(batch, k_pts, 3, want_experts=True, prompt=prompt)
            by = decode_bytes(n, r["distinct"], batch, r["ctx_tokens"], EL)
            out["points"][name] = round(r["tok_s"], 1)
            out["points_frac"][name] = round(by / (r["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
    if args.kernel_table:
        kernel_table(tq, model, rng, V, args.batch, args.kernel_table)
    print(json.dumps(out))
    return 0


def kernel_table(tq, model, rng, V, batch, path):
    """Per-kernel device time of 4 decode steps at context 2,048 and of one 2,048-token prefill."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    eng = tq.Engine(model, max_tokens=batch * CONTEXT, max_slots=batch)
    seqs = [eng.open() for _ in range(batch)]
    for g0 in range(0, batch, 8):
        eng.step([tq.StepEntry(s, rng.integers(0, V, size=PROMPT).tolist(), []) for s in seqs[g0:g0 + 8]])
    step = lambda: eng.step([tq.StepEntry(s, [1], [0]) for s in seqs])
    step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(4):
            step()
        torch.cuda.synchronize()
    text = "== 4 decode steps, batch %d, context %d ==\n" % (batch, PROMPT)
    text += prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70)
    for s in seqs:
        eng.close(s)
    s = eng.open()
    toks = rng.integers(0, V, size=PROMPT).tolist()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step([tq.StepEntry(s, toks, [PROMPT - 1])])
        torch.cuda.synchronize()
    text += "\n== prefill of one %d-token prompt ==\n" % PROMPT
    text += prof.key_averages().table(sort_by="cuda_time_total", row_limit=25, max_name_column_width=70)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    open(path, "w").write(text)


if __name__ == "__main__":
    sys.exit(main())
