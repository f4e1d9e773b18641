"""The command line's built-in measurements, after the reference's --bench-prefill and
--bench-memory modes (tools/quant.c:804-859 and :726-797): prompt speed, and decode speed at
growing context lengths.  Synthetic token ids; times from CUDA events."""
from __future__ import annotations

import sys

import torch

from .step import StepEntry


def device_peaks():
    """(GB/s, bf16 TFLOP/s) to hold the profile's figures against: $TQ_PEAK_GBS and $TQ_PEAK_TFLOPS if set (for
    instance from a measurement of this machine), else the B200's nominal 7,700 GB/s and 2,250 TFLOP/s."""
    import os
    return float(os.environ.get("TQ_PEAK_GBS", 7700.0)), float(os.environ.get("TQ_PEAK_TFLOPS", 2250.0))


def _time_ms(fn) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


def bench_prefill(m, n_tokens: int = 0, file=sys.stderr) -> float:
    eng = m.engine
    n = n_tokens or min(2048, m.context_length)
    toks = [i % eng.model.vocab_size for i in range(n)]
    best = float("inf")
    for _ in range(3):
        seq = eng.open()
        ms = _time_ms(lambda: eng.step([StepEntry(seq, toks, [n - 1])]))
        eng.close(seq)
        best = min(best, ms)
    print(f"PREFILL_CSV:{n},{best:.3f},{n / best * 1e3:.1f}", file=file)
    print(f"prefill: {n} tokens in {best:.2f} ms ({n / best * 1e3:.0f} tok/s)", file=file)
    return n / best * 1e3


def bench_memory(m, file=sys.stderr) -> None:
    eng = m.engine
    V = eng.model.vocab_size
    for ctx in (16, 64, 256, 1024, 4096, 16384):
        if ctx + 20 > m.context_length:
            break
        seq = eng.open()
        eng.step([StepEntry(seq, [i % V for i in range(ctx)], [])])
        ms = _time_ms(lambda: [eng.step([StepEntry(seq, [1], [0])]) for _ in range(20)])
        eng.close(seq)
        print(f"BENCH_CSV:{ctx},{20 / ms * 1e3:.2f}", file=file)
        print(f"decode at context {ctx}: {20 / ms * 1e3:.1f} tok/s", file=file)


BUCKETS = ("matmul", "moe", "attn", "other")      # the reference's, without its recurrent and conv1d ones


def bucket_of(kernel_name: str) -> str:
    """The profile bucket of a device kernel, by its name: dense products (the library's GEMMs) are 'matmul' as in the
    reference, where they go through tq_matmul; router, layout, experts and their sum are 'moe'; the fused
    bias/rotary/cache write and the attention kernels are 'attn'; norms, embedding, sampling and copies 'other'."""
    n = kernel_name.lower()
    if any(k in n for k in ("gemm_tc", "router", "moe_", "grouped_gemm", "gather_rows")):
        return "moe"
    if "attention" in n or "qkv_rope" in n:
        return "attn"
    if any(k in n for k in ("nvjet", "gemm", "gemv", "cutlass", "cublas", "splitk")):
        return "matmul"
    return "other"


def profile_generation(m, prompts, hbm_gbs: float, tflops: float, file=sys.stderr):
    """Generates for `prompts` under the device profiler and prints, per phase (the prompts' step, the decode
    steps), the share and the time per token of each bucket as the reference's --profile does
    (src/engine/tq_transformer.c:2994-3021), and what the reference does not: each bucket's bytes and operations
    against the peaks.  Kernel times are device times of kernels launched one after another (no CUDA graphs;
    TQ_NO_PDL=1 in the environment keeps a kernel's time free of its wait for the one before)."""
    from torch.profiler import ProfilerActivity, profile
    eng = m.engine
    results = {}
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        outs = m.generate_batch(prompts)
        torch.cuda.synchronize()
    st = m.last_stats
    times = {b: 0.0 for b in BUCKETS}
    for ev in prof.key_averages():
        t = getattr(ev, "self_device_time_total", None)
        if t is None:
            t = getattr(ev, "self_cuda_time_total", 0.0)
        if t:
            times[bucket_of(ev.key)] += t * 1e-6
    total = sum(times.values())
    n_tok = max(1, st.generated_tokens)
    if total > 0:
        print(f"[Profile {n_tok} tok] " + " ".join(f"{b}={times[b] / total * 100:.1f}%" for b in BUCKETS)
              + f" | per-tok: {total / n_tok * 1e3:.2f}ms (" + " ".join(f"{b}={times[b] / n_tok * 1e3:.2f}" for b in BUCKETS) + ")",
              file=file)
    # what the steps had to read and compute: the prompts' step once, then one step per generated token
    batch = len(prompts)
    n_prompt = sum(len(p) for p in prompts)
    steps = max(1, st.steps - st.batches)
    work = {b: [0.0, 0.0] for b in BUCKETS}
    model = eng.model
    for bucket, (byt, fl) in model.step_work(n_prompt, n_prompt, batch).items():
        work[bucket if bucket in work else "other"][0] += byt
        work[bucket if bucket in work else "other"][1] += fl
    mean_kv = n_prompt + batch * steps / 2.0
    for bucket, (byt, fl) in model.step_work(batch, int(mean_kv)).items():
        work[bucket if bucket in work else "other"][0] += byt * steps
        work[bucket if bucket in work else "other"][1] += fl * steps
    for b in BUCKETS:
        byt, fl = work[b]
        if times[b] > 0 and (byt or fl):
            print(f"[Profile] {b}: {byt / 1e9:.2f} GB and {fl / 1e12:.3f} TFLOP in {times[b] * 1e3:.2f} ms = "
                  f"{byt / times[b] / 1e9:.0f} GB/s ({byt / times[b] / 1e9 / hbm_gbs * 100:.0f}% of {hbm_gbs:.0f}), "
                  f"{fl / times[b] / 1e12:.1f} TFLOP/s ({fl / times[b] / 1e12 / tflops * 100:.1f}% of {tflops:.0f})", file=file)
    results.update(times=times, work=work, outs=outs)
    return results
