"""Host-side bookkeeping of the cache: pages of key/value storage and slots of fixed-size state.

Nothing here touches a device, so the rules can be tested on a CPU: a page or a slot is held by
at most one sequence, is given back exactly once, and none is lost.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence


class CacheFull(RuntimeError):
    """The cache cannot hold what a step asks for."""


class CacheMisuse(RuntimeError):
    """A page or slot was given back twice, or by someone who does not hold it."""


class IndexPool:
    """A pool of indices 0..n-1.  Freed indices are used again, most recently freed first."""

    def __init__(self, n: int, what: str):
        self.n, self.what = int(n), what
        self._free: List[int] = list(range(self.n - 1, -1, -1))
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def take_many(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}s wanted, {len(self._free)} of {self.n} are free")
        return [self.take() for _ in range(count)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheMisuse(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheMisuse(f"{self.what} {i} is given back but not held")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return self._held[i]


class Sequence_:
    """One live sequence: its slot, its length and, for each group of layers, its pages
    (index = position // page_size; None where a windowed group has given a page back)."""

    def __init__(self, seq_id: int, slot: int, n_groups: int):
        self.id = seq_id
        self.slot = slot
        self.length = 0
        self.pages: List[List[Optional[int]]] = [[] for _ in range(n_groups)]
        self.open = True


class CacheBook:
    """Pages and slots of all groups.  ``windows[g]`` is the window of group g (0: keeps all)."""

    def __init__(self, n_pages: Sequence[int], windows: Sequence[int], page_size: int, max_slots: int):
        assert len(n_pages) == len(windows)
        self.page_size = int(page_size)
        self.windows = [int(w) for w in windows]
        self.pools = [IndexPool(n, f"page of group {g}") for g, n in enumerate(n_pages)]
        self.slots = IndexPool(max_slots, "sequence slot")
        self._next_id = 0
        self.live: Dict[int, Sequence_] = {}

    def open(self) -> Sequence_:
        s = Sequence_(self._next_id, self.slots.take(), len(self.pools))
        self._next_id += 1
        self.live[s.id] = s
        return s

    def pages_needed(self, seq: Sequence_, n_new: int) -> List[int]:
        total = -(-(seq.length + n_new) // self.page_size)
        return [max(0, total - len(p)) for p in seq.pages]

    def reserve(self, seq: Sequence_, n_new: int) -> None:
        """Pages so that positions length .. length+n_new-1 can be written.  All or nothing."""
        self._check_open(seq)
        need = self.pages_needed(seq, n_new)
        for g, c in enumerate(need):
            if c > self.pools[g].n_free:
                raise CacheFull(f"sequence {seq.id} needs {c} more pages of {self.page_size} tokens in group {g} "
                                f"for {seq.length}+{n_new} tokens, {self.pools[g].n_free} of {self.pools[g].n} are free")
        for g, c in enumerate(need):
            seq.pages[g].extend(self.pools[g].take_many(c))

    def reserve_all(self, seqs: Sequence[Sequence_], n_new: Sequence[int]) -> None:
        """Reserve for a whole step, or for none of it."""
        for g in range(len(self.pools)):
            want = sum(self.pages_needed(s, n)[g] for s, n in zip(seqs, n_new))
            if want > self.pools[g].n_free:
                raise CacheFull(f"the step needs {want} more pages of {self.page_size} tokens in group {g}, "
                                f"{self.pools[g].n_free} of {self.pools[g].n} are free")
        for s, n in zip(seqs, n_new):
            self.reserve(s, n)

    def commit(self, seq: Sequence_, n_new: int) -> None:
        """The step wrote n_new tokens.  A windowed group gives back the pages no later query can see:
        a query at position p >= length reads positions >= p + 1 - window."""
        self._check_open(seq)
        seq.length += n_new
        for g, w in enumerate(self.windows):
            if w <= 0:
                continue
            first_visible = max(0, seq.length + 1 - w)
            for i in range(min(first_visible // self.page_size, len(seq.pages[g]))):
                if seq.pages[g][i] is not None:
                    self.pools[g].give_back(seq.pages[g][i])
                    seq.pages[g][i] = None

    def close(self, seq: Sequence_) -> None:
        self._check_open(seq)
        for g, pages in enumerate(seq.pages):
            for p in pages:
                if p is not None:
                    self.pools[g].give_back(p)
            pages.clear()
        self.slots.give_back(seq.slot)
        seq.open = False
        del self.live[seq.id]

    def _check_open(self, seq: Sequence_) -> None:
        if not seq.open or self.live.get(seq.id) is not seq:
            raise CacheMisuse(f"sequence {seq.id} is not live in this cache (closed twice?)")

    def check_invariants(self) -> None:
        """Every page and slot is either free or held by exactly one live sequence."""
        for g, pool in enumerate(self.pools):
            held = [p for s in self.live.values() for p in s.pages[g] if p is not None]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held twice")
            if len(held) != pool.n_held:
                raise AssertionError(f"group {g}: {pool.n_held} pages are out but sequences hold {len(held)}")
        slots = [s.slot for s in self.live.values()]
        if len(slots) != len(set(slots)) or len(slots) != self.slots.n_held:
            raise AssertionError("slots held do not match live sequences")
