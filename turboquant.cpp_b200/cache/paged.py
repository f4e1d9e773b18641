"""The cache on the device: pages of keys and values for every layer that keeps some, in groups
of layers with equal needs, and an area of fixed-size state per sequence slot.

The reference keeps one sequence's keys and values as [layer][position][kv heads * head size]
arrays written at the token's position (src/engine/tq_transformer.c:210-227, 1371, 1452-1455) and
its recurrent layers' fixed-size state in the same object, zeroed at creation
(include/turboquant/tq_engine.h:329-330; src/engine/tq_transformer.c:291-313).  Here:

* a *group* is the set of schedule entries whose mixers have the same KVNeed (heads, head size,
  window).  Each group has its own pool of pages and each sequence its own page list per group,
  so layers that keep every key and layers that keep a window of them are stored apart; a
  windowed group gives pages back as they fall out of every later query's sight.
* an entry's storage is one tensor [pages, 2 (K, V), kv heads, page_size, head size].
* a sequence holds a *slot*: its row in every state tensor [max_slots, *shape].  The row is
  zeroed when the slot is taken.  Slots and pages are given back when the sequence is closed and
  are used again by later sequences.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KVNeed, LayerCache, StateNeed
from .allocator import CacheBook, CacheFull, Sequence_

PAGE_SIZE = 64


class PagedCache:
    def __init__(self, kv_needs: Sequence[Optional[KVNeed]], state_needs: Sequence[Optional[StateNeed]],
                 cache_of: Sequence[Optional[int]], max_tokens: int, dtype: torch.dtype, device,
                 max_slots: Optional[int] = None, page_size: int = PAGE_SIZE,
                 pages_per_group: Optional[Dict[KVNeed, int]] = None):
        """kv_needs/state_needs/cache_of: one item per entry of the model's layer schedule.
        max_tokens: the most tokens live sequences hold together, each sequence's count rounded up
        to a multiple of page_size."""
        self.page_size = int(page_size)
        self.device = torch.device(device)
        self.dtype = dtype
        n_pages = max(1, -(-int(max_tokens) // self.page_size))
        self.max_slots = int(max_slots) if max_slots is not None else min(n_pages, 1024)
        self.groups: List[KVNeed] = []
        self.entry_group: List[Optional[int]] = []
        for i, need in enumerate(kv_needs):
            src = cache_of[i]
            if src is not None:
                self.entry_group.append(None)      # filled below from its source
                continue
            if need is None:
                self.entry_group.append(None)
                continue
            if need not in self.groups:
                self.groups.append(need)
            self.entry_group.append(self.groups.index(need))
        for i, src in enumerate(cache_of):
            if src is not None:
                self.entry_group[i] = self.entry_group[src]
        counts = [(pages_per_group or {}).get(g, n_pages) for g in self.groups]
        self.book = CacheBook(counts, [g.window for g in self.groups], self.page_size, self.max_slots)
        self.kv: List[Optional[torch.Tensor]] = []
        for i, need in enumerate(kv_needs):
            if need is None or cache_of[i] is not None:
                self.kv.append(None)
                continue
            g = self.entry_group[i]
            self.kv.append(torch.zeros((counts[g], 2, need.n_kv_heads, self.page_size, need.head_dim),
                                       dtype=dtype, device=self.device))
        for i, src in enumerate(cache_of):
            if src is not None:
                self.kv[i] = self.kv[src]
        self.cache_of = list(cache_of)
        self.state: List[Optional[torch.Tensor]] = [
            None if n is None else torch.zeros((self.max_slots,) + tuple(n.shape), dtype=n.dtype, device=self.device)
            for n in state_needs]

    # ---- sequences ------------------------------------------------------------------------------
    def open(self) -> Sequence_:
        seq = self.book.open()
        for s in self.state:
            if s is not None:
                s[seq.slot].zero_()
        return seq

    def close(self, seq: Sequence_) -> None:
        self.book.close(seq)

    def reserve(self, seqs: Sequence[Sequence_], n_new: Sequence[int]) -> None:
        self.book.reserve_all(seqs, n_new)

    def commit(self, seqs: Sequence[Sequence_], n_new: Sequence[int]) -> None:
        for s, n in zip(seqs, n_new):
            self.book.commit(s, n)

    # ---- what a step sees -----------------------------------------------------------------------
    def page_tables(self, seqs: Sequence[Sequence_]) -> List[np.ndarray]:
        """Per group an int32 array [n_seqs, width]: the pages of each sequence (-1: none)."""
        out = []
        for g in range(len(self.groups)):
            width = max(1, max((len(s.pages[g]) for s in seqs), default=1))
            t = np.full((len(seqs), width), -1, dtype=np.int32)
            for i, s in enumerate(seqs):
                pages = s.pages[g]
                if pages:
                    t[i, :len(pages)] = [(-1 if p is None else p) for p in pages]
            out.append(t)
        return out

    def layer_caches(self, device_tables: Sequence[torch.Tensor]) -> List[LayerCache]:
        out = []
        for i in range(len(self.kv)):
            g = self.entry_group[i]
            out.append(LayerCache(kv=self.kv[i], page_table=None if g is None else device_tables[g],
                                  page_size=self.page_size, writes=self.cache_of[i] is None,
                                  state=self.state[i]))
        return out

    def bytes_per_token(self) -> int:
        """Key/value bytes one token adds across all layers that keep a cache."""
        el = torch.empty((), dtype=self.dtype).element_size()
        return sum(2 * t.shape[2] * t.shape[4] * el for i, t in enumerate(self.kv)
                   if t is not None and self.cache_of[i] is None)
