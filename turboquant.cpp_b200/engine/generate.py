"""The generation loop: batches of unequal prompts, stop tokens, sequences that end earlier, and
as many batches one after another as there are requests.

The reference generates one sequence per call: prompt, first sample, then a loop of
{stop check, forward, sample} until max_tokens (src/engine/tq_generate.c:167-643; end-of-sequence
ids at :426-438, the loop at :441-605).  Its text stops are not carried over: stop tokens are a
set the caller gives (the configuration's eos ids by default).  Its repetition penalty (:586-600)
is the sampler's: a sampler that penalizes is handed each request's tokens so far.  Its detector of
repetition loops (:610-630) is LoopDetector below, off unless GenParams.detect_loops asks for it.

The decisions — which requests share a batch, when a sequence ends, when a batch ends — are host
code over an engine-like object, so they are tested on a CPU with a stand-in engine.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

from ..cache.allocator import CacheFull


@dataclass
class GenParams:
    max_new_tokens: int = 256
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 42
    stop_token_ids: Tuple[int, ...] = ()
    rep_penalty: float = 1.0         # > 1: the sampler lowers the logits of the last rep_window tokens
    rep_window: int = 32
    detect_loops: bool = False       # end a request whose last four tokens have come up three times before


@dataclass
class GenResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # 'stop' | 'length' | 'context' | 'loop'


@dataclass
class GenStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    batches: int = 0
    steps: int = 0


class LoopDetector:
    """The reference's detector of repetition loops (src/engine/tq_generate.c:370-384, 610-630): after every
    sampled token but a request's first, the last four tokens (the tail of the prompt counts) are hashed
    (h = h * 31 + token, 32 bits) and compared with the hashes of the 64 draws before; three matches mean a
    loop.  The reference then stops without emitting the token that closed the loop."""

    def __init__(self, prompt: Sequence[int], window: int = 32):
        self.recent = list(prompt)[-max(0, min(int(window), 128)):] if window > 0 else []
        self.hashes: List[int] = []
        self.first = True

    def push(self, token: int) -> bool:
        """Takes the newly sampled token; True if it closes a loop."""
        self.recent.append(int(token))
        del self.recent[:-128]
        if self.first:
            self.first = False
            return False
        if len(self.recent) < 4:
            return False
        h = 0
        for t in self.recent[-4:]:
            h = (h * 31 + (t & 0xFFFFFFFF)) & 0xFFFFFFFF
        matches = self.hashes[-64:].count(h)
        self.hashes.append(h)
        del self.hashes[:-64]
        return matches >= 3


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int, capacity_tokens: int,
                 max_slots: int, page_size: int, max_position: int) -> List[List[int]]:
    """Splits requests, in order, into batches that fit the cache: a request is counted with the
    most tokens it can come to hold, rounded up to whole pages."""
    if max_batch < 1:
        raise ValueError("max_batch must be at least 1")
    budget = capacity_tokens // page_size
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {i} has an empty prompt")
        if n > max_position:
            raise ValueError(f"request {i}: prompt of {n} tokens exceeds the model's {max_position} positions")
        need = -(-min(n + max_new_tokens, max_position) // page_size)
        if -(-n // page_size) > budget:
            raise CacheFull(f"request {i}: prompt of {n} tokens does not fit a cache of {capacity_tokens} tokens")
        need = min(need, budget)     # alone it may run until the cache is full
        if cur and (len(cur) >= min(max_batch, max_slots) or used + need > budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


def generate(engine, sampler, prompts: Sequence[Sequence[int]], params: GenParams, max_batch: int = 64,
             on_tokens: Optional[Callable[[List[int], List[int]], None]] = None,
             stats: Optional[GenStats] = None, sync: Optional[Callable[[], None]] = None) -> List[GenResult]:
    """Generates a continuation for every prompt.

    engine:   open(), close(seq), step(entries) -> logits rows, make_entry(seq, tokens, want),
              capacity_tokens, max_slots, page_size, max_position; optionally can_step_ahead, step_ahead(seqs,
              sampled tokens) -> logits rows, commit_ahead(), drop_ahead(), token_reader(n); optionally
              tokens_to_host(sampled tokens) -> list, which may raise if the step's kernels reported a fault (the
              tokens are then neither appended nor told)
    sampler:  sample(logits, request indices, token indices) -> one token per row (anything with .tolist());
              if it has `penalizes` set, also recent=[tokens of each request so far, prompt first]
    on_tokens(request indices, tokens) is called after every step with that step's new tokens.
    A stop token ends its sequence and is part of the output; with params.detect_loops a token that closes a
    repetition loop ends its sequence and is not (finish_reason 'loop').

    An engine that can (`can_step_ahead`) is kept one decode step ahead of the host: the next step is launched
    from the samples while they are still on the device, and the host reads them meanwhile.  If a sequence
    turns out to have ended, that step is dropped and run again without it, so the results are the same."""
    stats = stats if stats is not None else GenStats()
    sync = sync or (lambda: None)
    results = [GenResult() for _ in prompts]
    stop = set(int(t) for t in params.stop_token_ids)
    if params.max_new_tokens <= 0:
        for r in results:
            r.finish_reason = "length"
        return results
    batches = plan_batches([len(p) for p in prompts], params.max_new_tokens, max_batch, engine.capacity_tokens,
                           engine.max_slots, engine.page_size, engine.max_position)
    for batch in batches:
        stats.batches += 1
        live = {i: engine.open() for i in batch}
        loops = {i: LoopDetector(prompts[i], params.rep_window) for i in batch} if params.detect_loops else None
        ahead = None                                     # (request order, logits) of a step launched ahead
        try:
            # the prompts, whole, in one step; logits at each prompt's last token
            t0 = time.perf_counter()
            order = list(batch)
            logits = engine.step([engine.make_entry(live[i], list(prompts[i]), [len(prompts[i]) - 1]) for i in order])
            penalizes = bool(getattr(sampler, "penalizes", False))

            def so_far(rows):                            # what a penalizing sampler looks back at
                return {"recent": [list(prompts[i]) + results[i].tokens for i in rows]} if penalizes else {}
            to_host = getattr(engine, "tokens_to_host", None) or (lambda t: t.tolist())
            into = getattr(engine, "sample_into", None)      # optional: the engine's own place for a step's samples

            def sample(logits, rows, steps):
                kw = so_far(rows)
                if into is not None:
                    kw["out"] = into(len(rows))
                return sampler.sample(logits, rows, steps, **kw)
            new_dev = sample(logits, order, [0] * len(order))
            new = to_host(new_dev)
            sync()
            stats.prefill_seconds += time.perf_counter() - t0
            stats.prompt_tokens += sum(len(prompts[i]) for i in order)
            stats.steps += 1
            t0 = time.perf_counter()
            can_ahead = bool(getattr(engine, "can_step_ahead", False))
            reader = engine.token_reader(len(order)) if can_ahead else None
            while True:
                nxt: List[Tuple[int, int]] = []
                told_idx: List[int] = []
                told_tok: List[int] = []
                for i, tok in zip(order, new):
                    res = results[i]
                    if loops is not None and loops[i].push(int(tok)):
                        res.finish_reason = "loop"       # the token that closed the loop is not part of the output
                        engine.close(live.pop(i))
                        continue
                    res.tokens.append(int(tok))
                    told_idx.append(i)
                    told_tok.append(int(tok))
                    stats.generated_tokens += 1
                    if int(tok) in stop:
                        res.finish_reason = "stop"
                    elif len(res.tokens) >= params.max_new_tokens:
                        res.finish_reason = "length"
                    elif live[i].length + 1 > engine.max_position:
                        res.finish_reason = "context"
                    else:
                        nxt.append((i, int(tok)))
                        continue
                    engine.close(live.pop(i))            # the sequence ends: its slot and pages go back
                if on_tokens is not None and told_idx:
                    on_tokens(told_idx, told_tok)
                if not nxt:
                    break
                if ahead is not None and ahead[0] == [i for i, _ in nxt]:
                    engine.commit_ahead()                # nobody ended: the step launched ahead is this step
                    logits = ahead[1]
                    ahead = None
                else:
                    if ahead is not None:                # somebody ended: that step is void
                        ahead = None
                        engine.drop_ahead()
                    order = [i for i, _ in nxt]
                    try:
                        logits = engine.step([engine.make_entry(live[i], [tok], [0]) for i, tok in nxt])
                    except CacheFull:
                        for i in order:                  # no room for one more token each
                            results[i].finish_reason = "context"
                            engine.close(live.pop(i))
                        break
                new_dev = sample(logits, order, [len(results[i].tokens) for i in order])
                stats.steps += 1
                # launch the step after this one now, unless a sequence is sure to end with this token
                if can_ahead and all(len(results[i].tokens) + 1 < params.max_new_tokens
                                     and live[i].length + 1 <= engine.max_position for i in order):
                    arrived = reader.start(new_dev)
                    try:
                        ahead = (list(order), engine.step_ahead([live[i] for i in order], new_dev))
                    except CacheFull:
                        ahead = None
                    new = arrived()
                else:
                    new = to_host(new_dev)
            sync()
            stats.decode_seconds += time.perf_counter() - t0
        finally:
            if ahead is not None:                        # the batch ended, or an error, before the step's fate
                engine.drop_ahead()
            for seq in live.values():
                engine.close(seq)
    return results
