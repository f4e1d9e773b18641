"""Interfaces of the parts a model is put together from.

A decoder is a list of blocks; a block arranges a mixer (attention here) and
a feed-forward (dense or experts) around norms; a mixer may use a position
encoding.  Each part takes its sizes and constants as parameters, names the
tensors it needs, says what it needs from the cache, and runs on the tokens
of one step.  No part knows which model it is in, so a model chooses its
parts layer by layer, and one model can mix different mixers and
feed-forwards.

The reference has the same division only implicitly, as branches inside one
forward function (src/engine/tq_transformer.c:2410-2830: per-layer choice of
attention or recurrent mixer :2517-2551 and of MoE or dense feed-forward
:2681-2824).

Interfaces
----------
Part            weight_specs() -> [WeightSpec]; bind(store); kernels() -> names of kernel files
Norm            forward(x, out_dtype, rows, add) -> xn; add_forward(x, y) -> xn (x += y in fp32, then the norm)
PositionEncoding  tables() -> (cos, sin, pairing) or None; apply(q, k, positions)
Mixer           cache_need() -> KVNeed | None; state_need() -> StateNeed | None; capturable() -> bool;
                forward(xn, ctx, cache) -> y [T, hidden]
FeedForward     capturable() -> bool; forward(xn, ctx) -> y [T, hidden]
Block           cache_need(); state_need(); capturable(); forward(x, pending, ctx, cache) -> (x, pending):
                pending is a sub-layer output not yet added to the residual stream x (the sum is fused
                into the next norm).  A model talks to its blocks only through this interface.

capturable(): whether the part's forward can be recorded into a CUDA graph for decode steps: it reads
everything that changes from step to step from device tensors of the StepContext (positions, slots, page
tables, …), never from its host fields, and never synchronises.  One part that says no keeps the model's
decode steps out of graphs; nothing else changes.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..weights.loader import WeightSpec, WeightStore


@dataclass(frozen=True)
class KVNeed:
    """What a mixer needs from the key/value cache.  Layers with equal needs share a group of
    storage.  window = 0: every position is kept; window = w: positions older than the last w may
    be given back."""
    n_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size (one tensor of `shape` per sequence, zero at its start)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one entry of the layer schedule sees of the cache during a step."""
    kv: Optional[torch.Tensor] = None            # [pages, 2, n_kv_heads, page_size, head_dim]
    page_table: Optional[torch.Tensor] = None    # [n_seqs, width] int32, the group's pages per sequence
    page_size: int = 0
    writes: bool = True                          # False: reads another entry's cache, writes nothing
    state: Optional[torch.Tensor] = None         # [max_slots, *StateNeed.shape]


@dataclass
class StepContext:
    """The tokens of one step.  Sequences are packed one after another: token i belongs to sequence
    seq_of_token[i] (an index into this step's batch) and sits at absolute position positions[i]."""
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor            # [T] int32
    positions: torch.Tensor         # [T] int32
    seq_of_token: torch.Tensor      # [T] int32
    cu_seqlens: torch.Tensor        # [B+1] int32
    seq_start: torch.Tensor         # [B] int32: tokens each sequence held before this step
    slots: torch.Tensor             # [B] int32: row of each sequence in the fixed-size state area
    want_rows: torch.Tensor         # [n_want] int32: rows whose logits are wanted
    n_want: int
    max_q_len: int                  # longest run of new tokens among the sequences
    max_kv_len: int                 # longest sequence after this step
    act_dtype: torch.dtype          # dtype of activation tensors between kernels
    device: torch.device
    # host copies, for parts that must walk sequences in order (stateful mixers)
    host_q_lens: Sequence[int] = ()
    host_slots: Sequence[int] = ()
    debug: Optional[Dict[str, Any]] = None      # tests: parts may record what they decided
    status: Optional[torch.Tensor] = None       # int32 [1]: kernels with bounded waits report here when one ran out


class Part:
    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, store: WeightStore) -> None:
        """Take the tensors named by weight_specs() from the store."""

    def kernels(self) -> List[str]:
        """Kernel files (csrc/<name>.cu) this part launches; they are built before the first step."""
        return []

    def step_work(self, n_tokens: int, kv_tokens: int) -> Dict[str, Tuple[float, float]]:
        """What a step of n_tokens tokens over sequences that hold kv_tokens tokens together has to do in this
        part, for the command line's profile: {bucket: (bytes it must read, floating-point operations)} with the
        reference's bucket names 'matmul', 'moe', 'attn' (src/engine/tq_transformer.c:65-72); anything else is
        'other'.  Parts that say nothing are counted as nothing."""
        return {}


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                add: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Norm of the rows of x (of x + add if add is given); with `rows`, of those rows only.
        x is not changed."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, y: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def tables(self):
        """(cos, sin, pairing) for kernels that rotate inside a fused pass, or None."""
        return None

    def prepare(self, device) -> None:
        """Build device tables."""

    def apply(self, q: torch.Tensor, k: Optional[torch.Tensor], positions: torch.Tensor) -> None:
        """Encode positions into q [T, nh, hd] and k [T, nkv, hd] in place (used by mixers
        that have no fused pass for this encoding)."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        """Per-sequence state of fixed size: the step hands the mixer `cache.state` [max_slots, *shape], zero at
        a sequence's start; row ctx.slots[i] belongs to the step's i-th sequence.  Every token must update it
        exactly once."""
        return None

    def capturable(self) -> bool:
        return True

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def capturable(self) -> bool:
        return True

    def forward(self, xn: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """One entry of a model's list of layers: the arrangement of a mixer, a feed-forward and norms around the
    residual stream.  The model asks a block what its layer needs from the cache and runs it; it never looks
    inside."""

    def cache_need(self) -> Optional[KVNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def capturable(self) -> bool:
        return True

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], ctx: StepContext,
                cache: LayerCache) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        raise NotImplementedError


# ---- registries of part kinds: a configuration can choose parts by name --------------------
MIXERS: Dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: Dict[str, Callable[..., FeedForward]] = {}
NORMS: Dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: Dict[str, Callable[..., PositionEncoding]] = {}


def _register(table: Dict[str, Any], what: str, name: str, factory: Any, replace: bool) -> None:
    if name in table and not replace:
        raise ValueError(f"{what} '{name}' is already registered")
    table[name] = factory


def register_mixer(name: str, factory: Any, replace: bool = False) -> None:
    _register(MIXERS, "mixer", name, factory, replace)


def register_feed_forward(name: str, factory: Any, replace: bool = False) -> None:
    _register(FEED_FORWARDS, "feed-forward", name, factory, replace)


def register_norm(name: str, factory: Any, replace: bool = False) -> None:
    _register(NORMS, "norm", name, factory, replace)


def register_position_encoding(name: str, factory: Any, replace: bool = False) -> None:
    _register(POSITION_ENCODINGS, "position encoding", name, factory, replace)


def _make(table: Dict[str, Any], what: str, kind: str, /, **kw: Any):
    if kind not in table:
        raise KeyError(f"{what} '{kind}' is not registered; registered: {', '.join(sorted(table)) or '(none)'}")
    return table[kind](**kw)


def make_mixer(kind: str, /, **kw: Any) -> Mixer:
    return _make(MIXERS, "mixer", kind, **kw)


def make_feed_forward(kind: str, /, **kw: Any) -> FeedForward:
    return _make(FEED_FORWARDS, "feed-forward", kind, **kw)


def make_norm(kind: str, /, **kw: Any) -> Norm:
    return _make(NORMS, "norm", kind, **kw)


def make_position_encoding(kind: str, /, **kw: Any) -> PositionEncoding:
    return _make(POSITION_ENCODINGS, "position encoding", kind, **kw)
