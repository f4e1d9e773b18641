"""The step function: one batch of sequences, the tokens each brings, logits at the wanted places.

A step runs only the tokens it is given, packed one sequence after another with no padding, on
top of what earlier steps left in the cache.  Sequences of one batch usually start together with
whole prompts of unequal lengths and then go on by one token each; the step itself accepts any
cut (a prompt in pieces, one token at a time).  The logits at a position do not depend on the cut
or on the batch beyond rounding.

The reference's step is one token of one sequence (`tq_forward(model, state, token, pos)`,
include/turboquant/tq_engine.h:529); its only multi-token path handles one sequence, dense layers
only, and returns the last row's logits (src/engine/tq_transformer.c:3049-3592, MoE refused at
:3066-3067).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import os

import numpy as np
import torch

from ..cache import CacheFull, PagedCache, Sequence_
from ..csrc.build import ensure_built, index_faults
from ..kernels._call import KernelError
from ..kernels.gemm_tc import GAVE_UP, check_status
from ..parts.base import StepContext
from .graph import DecodeGraphs


class StepError(ValueError):
    """A step that cannot run: bad token ids, places, or a sequence beyond the model's positions."""


@dataclass
class StepEntry:
    seq: Sequence_
    tokens: Sequence[int]
    want: Sequence[int] = ()      # places among `tokens` whose logits are asked for


FEED_TOKENS = 4      # where the tokens begin in an engine's feed buffer (the status word is element 0)


class TokenReader:
    """Brings a step's sampled tokens to the host without waiting for work queued behind them: two pinned
    buffers used in turn (allocated once: nothing is allocated or freed while steps are in flight), a copy and an
    event per step.  The engine's status word travels with the tokens: if a kernel gave up on a bounded wait,
    the tokens sampled from its output are never handed out."""

    def __init__(self, n: int, status: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None):
        """feed: the engine's [status, ..., tokens] buffer; samples that lie in it travel with the status word in
        one copy, on a stream of the reader's own, so that the step queued behind them does not wait for the copy."""
        self.bufs = [torch.empty(FEED_TOKENS + max(1, n) + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.turn = 0
        self.status = status
        self.feed = feed
        self.side = torch.cuda.Stream(device=feed.device) if feed is not None else None

    def _withheld(self):
        self.status.zero_()
        raise KernelError("step: " + GAVE_UP + "; the tokens sampled from it are withheld")

    def start(self, tokens_dev):
        """Starts the copy and returns the function that waits for it and gives the tokens.  Call that function
        before the next sampling: samples in the engine's feed buffer are overwritten by it."""
        self.turn ^= 1
        n = tokens_dev.numel()
        host = self.bufs[self.turn]
        done = torch.cuda.Event()
        if (self.feed is not None and tokens_dev.dtype == torch.int32
                and tokens_dev.data_ptr() == self.feed.data_ptr() + 4 * FEED_TOKENS):
            sampled = torch.cuda.Event()
            sampled.record()
            with torch.cuda.stream(self.side):
                self.side.wait_event(sampled)
                host[:FEED_TOKENS + n].copy_(self.feed[:FEED_TOKENS + n], non_blocking=True)
                done.record()

            def wait():
                done.synchronize()
                if int(host[0]) != 0:
                    self._withheld()
                return host[FEED_TOKENS:FEED_TOKENS + n].tolist()
            return wait
        host[:n].copy_(tokens_dev, non_blocking=True)
        if self.status is not None:
            host[n:n + 1].copy_(self.status, non_blocking=True)
        done.record()

        def wait():
            done.synchronize()
            if self.status is not None and int(host[n]) != 0:
                self._withheld()
            return host[:n].tolist()
        return wait


class Engine:
    """A model, its cache and the step function."""

    def __init__(self, model, max_tokens: int, max_slots: Optional[int] = None, device="cuda:0",
                 use_graphs: Optional[bool] = None, record_routing: bool = False):
        """record_routing: decode steps captured into CUDA graphs keep what the parts record into the step's
        `debug` (the experts chosen) in memory of the graph, so that setting `engine.debug = {}` before a step
        fills it from the very launches that generation replays; without it, a step with `debug` set runs
        outside the graphs."""
        self.model = model
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device; there is no CPU path")
        self.act_dtype = model.dtype
        ensure_built(model.kernels())
        self.cache = PagedCache(model.cache_needs(), model.state_needs(), [e.cache_of for e in model.schedule],
                                max_tokens, self.act_dtype, self.device, max_slots=max_slots)
        self.debug: Optional[Dict[str, Any]] = None
        self.record_routing = bool(record_routing)
        # set by a kernel whose bounded wait ran out (one word per engine: a fault is seen by the engine it spoiled)
        # The status word and the place where a step's sampled tokens are put share one buffer, [status, 3 unused,
        # a token per slot]: the samples go to the host together with the word in one copy, and a decode graph reads
        # its step's tokens there, so between two decode steps the stream carries the sampling kernel and one copy
        # of the step's metadata, not six small operations with a gap of about ten microseconds before each.
        self.feed = torch.zeros(FEED_TOKENS + self.cache.max_slots, dtype=torch.int32, device=self.device)
        self.status = self.feed[0:1]
        self.steps_run = 0
        # widest page table a sequence can need; decode graphs keep tables of this width
        longest = min(self.model.max_position, max(self.capacity_tokens, self.cache.page_size))
        self.table_width = -(-longest // self.cache.page_size)
        if use_graphs is None:
            use_graphs = os.environ.get("TQ_NO_GRAPHS", "") in ("", "0")
        # a part that cannot run inside a captured step (it says so itself) keeps the whole model out of graphs
        self.graphs = DecodeGraphs(self) if use_graphs and model.capturable() else None
        self._stateless = all(n is None for n in model.state_needs())
        # TQ_DEBUG_LAYERS=1 (or =all): every step prints the residual stream's sum and sum of magnitudes after each
        # layer, for positions 0 and 1 (or all), in the manner of the reference's TQ_DEBUG_PREFILL
        # (src/engine/tq_transformer.c:2827-2831); such steps run outside the CUDA graphs
        self.layer_dump = os.environ.get("TQ_DEBUG_LAYERS", "")
        if self.layer_dump in ("0", ""):
            self.layer_dump = ""
        self._ahead = None                       # (sequences, tokens each) of a step launched ahead, if any
        self._reader: Optional[TokenReader] = None

    # ---- what the generation loop asks -----------------------------------------------------------
    @property
    def capacity_tokens(self) -> int:
        return min(p.n for p in self.cache.book.pools) * self.cache.page_size if self.cache.book.pools else 1 << 30

    @property
    def max_slots(self) -> int:
        return self.cache.max_slots

    @property
    def page_size(self) -> int:
        return self.cache.page_size

    @property
    def max_position(self) -> int:
        return self.model.max_position

    @staticmethod
    def make_entry(seq: Sequence_, tokens: Sequence[int], want: Sequence[int] = ()) -> "StepEntry":
        return StepEntry(seq, tokens, want)

    def check_kernels(self) -> None:
        """Raises if a tensor-core kernel gave up on one of its bounded waits since the last check
        (it synchronises the device; call it where results are brought to the host anyway)."""
        check_status(word=self.status)
        faults = index_faults()                 # kernels built with their index checks (TQ_DEBUG_INDEX=1) report here
        if faults:
            raise KernelError("a kernel was handed an index outside its tensor: " + "; ".join(faults))

    def release(self) -> None:
        """Gives back what the engine holds on the device besides the cache: its CUDA graphs."""
        self._ahead = None
        if self.graphs is not None:
            self.graphs.release()

    def warm_up(self, batch_sizes) -> List[int]:
        """Captures the decode graphs of these batch sizes now, with one step of one-token sequences that are
        closed again, so that generation meets no new size in the middle of a batch (the first step of a new size
        runs kernel by kernel, waits for the device and records the graph: tens of milliseconds).  Returns the
        sizes captured by this call; sizes that have their graph already cost nothing.  It stops quietly at the
        first size the free slots or pages do not hold."""
        done: List[int] = []
        if self.graphs is None or self.debug is not None or self.layer_dump:
            return done
        for B in sorted({int(b) for b in batch_sizes}):
            if B < 1:
                raise StepError(f"warm_up: batch size {B}")
            g = self.graphs.graphs.get(B)
            if g is not None and g.graph is not None:
                continue
            seqs: List[Sequence_] = []
            try:
                for _ in range(B):
                    seqs.append(self.open())
                self.step([StepEntry(s, [0], [0]) for s in seqs])
                done.append(B)
            except CacheFull:
                break
            finally:
                for s in seqs:
                    self.close(s)
        return done

    # ---- sequences ------------------------------------------------------------------------------
    def open(self) -> Sequence_:
        return self.cache.open()

    def close(self, seq: Sequence_) -> None:
        self.cache.close(seq)

    # ---- one step -------------------------------------------------------------------------------
    def _check(self, entries: Sequence[StepEntry]) -> None:
        V, maxpos = self.model.vocab_size, self.model.max_position
        seen = set()
        for e in entries:
            if e.seq.id in seen:
                raise StepError(f"sequence {e.seq.id} appears twice in one step")
            seen.add(e.seq.id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"sequence {e.seq.id} brings no token to the step")
            if e.seq.length + n > maxpos:
                raise StepError(f"sequence {e.seq.id} would reach {e.seq.length + n} tokens; the model's "
                                f"max_position_embeddings is {maxpos}")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"sequence {e.seq.id}: wanted place {w} is outside its {n} tokens")

    def _check_tokens(self, tokens: np.ndarray) -> None:
        V = self.model.vocab_size
        if tokens.size and (tokens.min() < 0 or tokens.max() >= V):
            bad = int(tokens[(tokens < 0) | (tokens >= V)][0])
            raise StepError(f"token id {bad} is outside the vocabulary (0..{V - 1})")

    def build_context(self, entries: Sequence[StepEntry]) -> Tuple[StepContext, List[torch.Tensor]]:
        """Packs the step's metadata and sends it to the device in one copy."""
        B = len(entries)
        q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int64)
        T = int(q_lens.sum())
        starts = np.array([e.seq.length for e in entries], dtype=np.int64)
        cu = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu[1:])
        tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64).reshape(-1) for e in entries])
        self._check_tokens(tokens)
        seq_of_token = np.repeat(np.arange(B, dtype=np.int64), q_lens)
        positions = np.arange(T, dtype=np.int64) - cu[:-1][seq_of_token] + starts[seq_of_token]
        want = np.array([cu[i] + w for i, e in enumerate(entries) for w in e.want], dtype=np.int64)
        slots = np.array([e.seq.slot for e in entries], dtype=np.int64)
        tables = self.cache.page_tables([e.seq for e in entries])
        fields = [tokens, positions, seq_of_token, cu, starts, slots, want] + [t.reshape(-1) for t in tables]
        sizes = [f.size for f in fields]
        packed = torch.from_numpy(np.concatenate(fields).astype(np.int32))
        if packed.numel():
            packed = packed.pin_memory()
        dev = packed.to(self.device, non_blocking=True)
        parts = torch.split(dev, sizes)
        dev_tables = [parts[7 + g].view(tables[g].shape) for g in range(len(tables))]
        ctx = StepContext(
            n_tokens=T, n_seqs=B, tokens=parts[0], positions=parts[1], seq_of_token=parts[2], cu_seqlens=parts[3],
            seq_start=parts[4], slots=parts[5], want_rows=parts[6], n_want=int(want.size),
            max_q_len=int(q_lens.max()), max_kv_len=int((starts + q_lens).max()), act_dtype=self.act_dtype,
            device=self.device, host_q_lens=[int(n) for n in q_lens], host_slots=[int(s) for s in slots],
            debug=self.debug, status=self.status)
        return ctx, dev_tables

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs one step.  Returns float32 logits [number of wanted places, vocab] on the device, in
        the order of the entries and of each entry's `want`; None if nothing is wanted."""
        if not entries:
            return None
        self._check(entries)
        seqs = [e.seq for e in entries]
        n_new = [len(e.tokens) for e in entries]
        self.cache.reserve(seqs, n_new)          # raises CacheFull before anything is written
        decode = all(n == 1 and len(e.want) == 1 for n, e in zip(n_new, entries))
        if self.layer_dump:
            return self._step_with_layer_dump(entries, seqs, n_new)
        with torch.cuda.device(self.device):
            if decode and self.graphs is not None and (self.debug is None or self.record_routing):
                self._check_tokens(np.asarray([e.tokens[0] for e in entries], dtype=np.int64))
                logits = self.graphs.step(entries)
                if self.debug is not None:
                    self.graphs.copy_debug(len(entries), self.debug)
            else:
                ctx, dev_tables = self.build_context(entries)
                logits = self.model.forward(ctx, self.cache.layer_caches(dev_tables))
        self.cache.commit(seqs, n_new)
        self.steps_run += 1
        return logits

    def _step_with_layer_dump(self, entries, seqs, n_new):
        import sys
        saved, self.debug = self.debug, dict(self.debug or {}, layer_sums=[])
        try:
            with torch.cuda.device(self.device):
                ctx, dev_tables = self.build_context(entries)
                logits = self.model.forward(ctx, self.cache.layer_caches(dev_tables))
            positions = ctx.positions.tolist()
            for layer, sums, mags in self.debug["layer_sums"]:
                sums, mags = sums.tolist(), mags.tolist()
                for t, pos in enumerate(positions):
                    if self.layer_dump == "all" or pos <= 1:
                        print(f"[fwd]   L{layer} pos={pos} final x sum={sums[t]:.9f} sumabs={mags[t]:.9f}", file=sys.stderr)
        finally:
            self.debug = saved
        self.cache.commit(seqs, n_new)
        self.steps_run += 1
        return logits

    # ---- a decode step launched before its input tokens have reached the host --------------------------
    @property
    def can_step_ahead(self) -> bool:
        """Decode steps can be launched from tokens that are still on the device (CUDA graphs, no per-sequence
        state that a dropped step would have changed)."""
        return self.graphs is not None and self.debug is None and self._stateless and not self.layer_dump

    def step_ahead(self, seqs: Sequence[Sequence_], tokens_dev: torch.Tensor) -> torch.Tensor:
        """Launches the decode step whose tokens are `tokens_dev` (int32, one per sequence, on the device: the
        samples of the step before) and returns its logits, without advancing the sequences: the caller reads the
        samples on the host meanwhile and then either keeps the step (`commit_ahead`) or, if a sequence turned
        out to have ended, drops it (`drop_ahead`) and steps again.  A dropped step leaves nothing behind: what it
        wrote into the cache lies beyond the sequences' lengths and is written again by the step that replaces it.
        The logits are the captured step's own buffer: they hold until the next decode step of this batch size."""
        if not self.can_step_ahead:
            raise StepError("this engine cannot launch a step ahead")
        if self._ahead is not None:
            raise StepError("a step launched ahead is still waiting to be kept or dropped")
        seqs = list(seqs)
        if len({s.id for s in seqs}) != len(seqs):
            raise StepError("a sequence appears twice in one step")
        for s in seqs:
            if s.length + 1 > self.model.max_position:
                raise StepError(f"sequence {s.id} would pass the model's max_position_embeddings")
        n_new = [1] * len(seqs)
        self.cache.reserve(seqs, n_new)          # raises CacheFull before anything is written
        with torch.cuda.device(self.device):
            logits = self.graphs.step_from_device(seqs, tokens_dev)
        self._ahead = (seqs, n_new)
        return logits

    def token_reader(self, n: int) -> TokenReader:
        """The engine's reader (pinned buffers for a token per slot, made once: pinning memory takes about a
        millisecond, which a short generation would notice)."""
        if self._reader is None:
            self._reader = TokenReader(max(n, self.max_slots), self.status, self.feed)
        return self._reader

    def sample_into(self, n: int) -> torch.Tensor:
        """Where a sampler should put the tokens of a step's n sequences (int32 on the device): from there they
        reach the host with the status word in one copy and the next decode step without one."""
        return self.feed[FEED_TOKENS:FEED_TOKENS + n]

    def tokens_to_host(self, tokens_dev: torch.Tensor) -> List[int]:
        """A step's sampled tokens as a list, after a look at the status word (one synchronisation for both)."""
        both = torch.cat([tokens_dev.to(torch.int32).reshape(-1), self.status]).tolist()
        if both[-1] != 0:
            self.status.zero_()
            raise KernelError("step: " + GAVE_UP + "; the tokens sampled from it are withheld")
        return both[:-1]

    def commit_ahead(self) -> None:
        seqs, n_new = self._ahead
        self._ahead = None
        self.cache.commit(seqs, n_new)
        self.steps_run += 1

    def drop_ahead(self) -> None:
        self._ahead = None
