"""CUDA graphs for decode steps.

A decode step (every sequence brings one token and wants its logits) launches a few hundred small
kernels; at small batches their launch cost, not their run time, bounds the step.  The step is
therefore captured once per batch size into a CUDA graph whose inputs are one static int32 buffer
(tokens, positions, page tables, …) and replayed with one copy into that buffer.  Everything a
kernel needs that changes from step to step lives in that buffer, never in a launch argument.
"""
from __future__ import annotations

import gc
from typing import Dict, List, Sequence

import numpy as np
import torch

from ..kernels import _call
from ..parts.base import StepContext


class DecodeGraph:
    """The captured forward pass of a decode step for one batch size."""

    def __init__(self, engine, batch: int):
        self.engine, self.batch = engine, batch
        cache = engine.cache
        self.widths = [engine.table_width for _ in cache.groups]
        B = batch
        sizes = [B, B, B, B + 1, B, B, B] + [B * w for w in self.widths]
        self.offsets = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
        total = int(self.offsets[-1])
        # two pinned staging buffers used in turn: a buffer is rewritten only after its copy has finished
        self.hosts = [torch.empty(total, dtype=torch.int32).pin_memory() for _ in range(2)]
        self.copied = [None, None]
        self.turn = 0
        self.dev = torch.zeros(total, dtype=torch.int32, device=engine.device)
        parts = [self.dev[self.offsets[i]:self.offsets[i + 1]] for i in range(len(sizes))]
        self.tables = [parts[7 + g].view(B, self.widths[g]) for g in range(len(self.widths))]
        self.ctx = StepContext(
            n_tokens=B, n_seqs=B, tokens=engine.sample_into(B), positions=parts[1], seq_of_token=parts[2], cu_seqlens=parts[3],
            seq_start=parts[4], slots=parts[5], want_rows=parts[6], n_want=B, max_q_len=1,
            max_kv_len=engine.table_width * cache.page_size, act_dtype=engine.act_dtype, device=engine.device,
            host_q_lens=[1] * B, host_slots=[], debug={} if engine.record_routing else None, status=engine.status)
        for host in self.hosts:              # constant parts of the buffer
            h = host.numpy()
            h[:] = 0
            h[self.offsets[2]:self.offsets[3]] = np.arange(B)
            h[self.offsets[3]:self.offsets[4]] = np.arange(B + 1)
            h[self.offsets[6]:self.offsets[7]] = np.arange(B)
        self.graph = None
        self.logits = None
        self.first_debug = None

    def fill(self, seqs, tokens: Sequence[int], with_tokens: bool = True) -> None:
        self.turn ^= 1
        if self.copied[self.turn] is not None:
            self.copied[self.turn].synchronize()
        host = self.hosts[self.turn]
        h, o, B = host.numpy(), self.offsets, self.batch
        lengths = [s.length for s in seqs]
        h[o[0]:o[1]] = tokens
        h[o[1]:o[2]] = lengths
        h[o[4]:o[5]] = lengths
        h[o[5]:o[6]] = [s.slot for s in seqs]
        for g, w in enumerate(self.widths):
            t = h[o[7 + g]:o[8 + g]].reshape(B, w)
            for i, s in enumerate(seqs):
                pages = s.pages[g]
                row = t[i]
                n = len(pages)
                row[:n] = [(-1 if p is None else p) for p in pages] if None in pages else pages
        self.dev.copy_(host, non_blocking=True)
        if with_tokens:
            self.engine.sample_into(B).copy_(host[o[0]:o[1]], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.copied[self.turn] = ev

    def run(self, seqs, tokens: Sequence[int], tokens_dev: torch.Tensor = None, own_logits: bool = True) -> torch.Tensor:
        """The step reads its tokens in the engine's feed buffer.  tokens_dev: the step's tokens as an int32 tensor
        on the device (the previous step's samples): nothing to do if they were sampled into the feed buffer, a
        device copy otherwise; without it the host's tokens are copied there.  own_logits: a copy of the logits
        (the captured step's buffer is written again by the next replay)."""
        eng = self.engine
        feed = eng.sample_into(self.batch)
        self.fill(seqs, tokens, with_tokens=tokens_dev is None)
        if tokens_dev is not None and tokens_dev.data_ptr() != feed.data_ptr():
            feed.copy_(tokens_dev, non_blocking=True)
        caches = eng.cache.layer_caches(self.tables)
        if self.graph is None:
            # the first step of this batch size runs eagerly (it also loads kernels and lets libraries
            # set up their workspaces); the same launches are then recorded, not run, for later steps
            logits = eng.model.forward(self.ctx, caches)
            torch.cuda.synchronize(eng.device)
            g = torch.cuda.CUDAGraph()
            if self.ctx.debug is not None:
                # this step's records are the eager run's; from the next step on, the captured launches'
                self.first_debug = {k: [t.clone() if isinstance(t, torch.Tensor) else t for t in v]
                                    for k, v in self.ctx.debug.items()}
                self.ctx.debug.clear()
            before = _call.LAUNCHES
            # no garbage collection while the stream is capturing: a collected object that owns device memory or
            # another CUDA graph (an engine that was dropped earlier) would free it in the middle of the capture,
            # which invalidates it
            gc.collect()
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(g, pool=self.engine.graphs.pool):
                    self.logits = eng.model.forward(self.ctx, caches)
            finally:
                if gc_was_on:
                    gc.enable()
            self.kernels = _call.LAUNCHES - before      # this library's kernels inside the graph
            _call.LAUNCHES = before
            self.graph = g
            return logits
        self.graph.replay()
        eng.graphs.replays += 1
        _call.LAUNCHES += self.kernels
        return self.logits.clone() if own_logits else self.logits


class DecodeGraphs:
    def __init__(self, engine):
        self.engine = engine
        self.graphs: Dict[int, DecodeGraph] = {}
        self.replays = 0                      # decode steps that ran as a replay of a captured graph
        # one memory pool for all batch sizes: replays are serial on one stream and every result is copied out
        # of the pool before the next replay, so the graphs can share their activations' memory
        self.pool = torch.cuda.graph_pool_handle()

    def copy_debug(self, batch: int, into: Dict) -> None:
        """Copies of what the parts recorded during the last step of this batch size."""
        g = self.graphs[batch]
        if g.first_debug is not None:
            into.update(g.first_debug)
            g.first_debug = None
            return
        for k, v in (g.ctx.debug or {}).items():
            into[k] = [t.clone() if isinstance(t, torch.Tensor) else t for t in v]

    def release(self) -> None:
        """Drops the captured graphs (and their memory) now, not when a garbage collector finds them."""
        for g in self.graphs.values():
            g.graph = g.logits = g.engine = None
        self.graphs.clear()

    def step(self, entries) -> torch.Tensor:
        B = len(entries)
        g = self.graphs.get(B)
        if g is None:
            g = self.graphs[B] = DecodeGraph(self.engine, B)
        return g.run([e.seq for e in entries], [int(e.tokens[0]) for e in entries])

    def step_from_device(self, seqs, tokens_dev: torch.Tensor) -> torch.Tensor:
        B = len(seqs)
        g = self.graphs.get(B)
        if g is None:
            g = self.graphs[B] = DecodeGraph(self.engine, B)
        return g.run(list(seqs), [0] * B, tokens_dev, own_logits=False)
