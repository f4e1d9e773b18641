"""Routed experts with a shared expert (src/engine/tq_moe.c:688-1059).

  router   logits = Wr x in fp32; p = softmax over all experts; the k most probable (ties to the
           lowest index); weights p[sel], divided by their sum if norm_topk.  The reference picks
           the k largest logits and takes a softmax over them (:600-682), i.e. the norm_topk case.
  experts  for each chosen e: o_e = Wd_e (silu(Wg_e x) * (Wu_e x)); y = sum w_e o_e (:864-1000)
  shared   y += sigmoid(w_sg . x) * shared_expert(x) (:1006-1058)

Tokens are copied into an expert-sorted layout, two grouped products run over it (gate|up with the
SiLU product fused, then down), and one pass sums each token's k rows and the shared expert in the
order above.  Router logits, softmax and the weighted sum are fp32 on both paths.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from ..kernels import elementwise as KE
from ..kernels import gemm_tc as KT
from ..kernels import moe as KM
from ..kernels.linear import linear
from ..weights.loader import WeightSpec, WeightStore
from .base import FeedForward, StepContext, register_feed_forward


def KA_resident(device) -> int:
    """SMs of the device (the tensor-core product runs up to two CTAs on each)."""
    from ..kernels.attention import resident_ctas
    return resident_ctas(device) // 4


def experts_touched(n_tokens: int, n_experts: int, top_k: int) -> float:
    """Distinct experts a step of n_tokens tokens reads under uniform routing."""
    return n_experts * (1.0 - ((n_experts - top_k) / n_experts) ** n_tokens)


def shared_down_shares(n_tokens: int, n_experts: int, top_k: int, intermediate: int, shared_intermediate: int,
                       hidden: int, token_tile: int, sms: int, router_first: bool, ratio: float = 14.0) -> int:
    """Into how many shares of K the shared expert's down projection (hidden x shared_intermediate, a CTA per 128
    output columns when whole) is cut in a decode step.
      * one or two tokens, or the router runs ahead of the shared expert: as many shares as fill the GPU
        (`k_splits_for`): the product is the longer of the layer's two chains;
      * while the routed experts of the step read less than about `ratio` times this product's bytes: two shares (four
        from 8,192 values of K on), so that it does not outlast the routed gate/up product beside it, whose persistent
        CTAs were counted on the SM slots it holds;
      * else one: shared out it would take SMs from the routed experts (3-10 % of the step).
    Measured on B200, tokens/s whole / in shares: A2.7B sizes batch 3: 1,246 / 1,277, 4: 1,423 / 1,481, 5: 1,666 /
    1,708, 6: 1,900 / 1,897, 8: 2,283 / 2,272; 57B-A14B sizes batch 1: 144 / 165, 3: 330 / 368, 4: 400 / 427, 6: 506 / 524."""
    S = shared_intermediate
    if token_tile > 64:
        return 1                                   # wide token tiles (prompts) fill the GPU as they are
    if n_tokens * top_k * intermediate <= 2 * S or router_first:
        return KT.k_splits_for(n_tokens, hidden, S, token_tile, 2 * sms)
    if experts_touched(n_tokens, n_experts, top_k) * 3 * intermediate <= ratio * S and S >= 32 * KT.BLOCK_K:
        return 2 if S < 128 * KT.BLOCK_K else 4
    return 1


def shared_rides_with_routed(n_tokens: int, shared_intermediate: int, sms: int) -> bool:
    """Whether a long step's shared expert has so few rounds of tiles (fewer than four per CTA pair in its gate/up
    product, at the widest token tile) that its tiles ride in the routed experts' launches."""
    units = -(-n_tokens // KT.TOKEN_TILES[-1]) * -(-shared_intermediate // KT.BLOCK_ROWS)
    return units < 4 * (sms // 2)


class MoEFeedForward(FeedForward):
    # steps with at least this many tokens (and too many pairs for the one-launch router) compute router logits on
    # tensor cores (measured on B200 at 64 tokens: +2.4 % on the step at the 57B-A14B sizes, +0.8 % at the A2.7B sizes)
    ROUTER_TC_MIN_TOKENS = int(os.environ.get("TQ_ROUTER_TC_MIN", "64"))
    SHARED_AFTER_ROUTER = {"": None, "0": False}.get(os.environ.get("TQ_SHARED_AFTER_ROUTER", ""), True)   # None: by the step's size
    # long steps: the shared expert's products in the launches of the routed experts' ("": by the step's size,
    # "0": never, "1": always, "spread": always, with the shared expert's tiles spread among the routed ones instead
    # of ahead of them)
    SHARED_IN_ROUTED_LAUNCH = os.environ.get("TQ_SHARED_DUAL", "")
    SHARED_DOWN_SPLIT_RATIO = float(os.environ.get("TQ_SHARED_DOWN_SPLIT_RATIO", "14"))

    def __init__(self, prefix: str, hidden: int, n_experts: int, top_k: int, intermediate: int,
                 norm_topk: bool, shared_intermediate: int = 0, shared_gate: bool = True):
        if n_experts < 1 or not 1 <= top_k <= n_experts:
            raise ValueError(f"experts '{prefix}': top-k {top_k} must be in 1..{n_experts}")
        if hidden < 1 or intermediate < 1 or shared_intermediate < 0:
            raise ValueError(f"experts '{prefix}': bad sizes {hidden}, {intermediate}, {shared_intermediate}")
        self.prefix, self.hidden = prefix, int(hidden)
        self.n_experts, self.top_k, self.intermediate = int(n_experts), int(top_k), int(intermediate)
        self.norm_topk, self.shared_intermediate = bool(norm_topk), int(shared_intermediate)
        self.shared_gate = bool(shared_gate) and shared_intermediate > 0
        self.w_router = self.w_shared_gate = self.w_router_packed = None
        self.w13 = self.w2 = None            # [E, 2I, H] (gate rows, up rows), [E, H, I]
        self.ws13 = self.ws2 = None          # shared expert [1, 2S, H], [1, H, S]

    def weight_specs(self) -> List[WeightSpec]:
        p, H, I, S = self.prefix, self.hidden, self.intermediate, self.shared_intermediate
        specs = [WeightSpec(p + "gate.weight", (self.n_experts, H))]
        for e in range(self.n_experts):
            q = f"{p}experts.{e}."
            specs += [WeightSpec(q + "gate_proj.weight", (I, H)), WeightSpec(q + "up_proj.weight", (I, H)),
                      WeightSpec(q + "down_proj.weight", (H, I))]
        if S > 0:
            q = p + "shared_expert."
            specs += [WeightSpec(q + "gate_proj.weight", (S, H)), WeightSpec(q + "up_proj.weight", (S, H)),
                      WeightSpec(q + "down_proj.weight", (H, S))]
            if self.shared_gate:
                specs.append(WeightSpec(p + "shared_expert_gate.weight", (1, H)))
        return specs

    def bind(self, store: WeightStore) -> None:
        p, H, I, S, E = self.prefix, self.hidden, self.intermediate, self.shared_intermediate, self.n_experts
        self.w_router = store.get(p + "gate.weight")
        # a tensor stored in 32 bits stays 32-bit: if any of the experts' tensors is kept in float32, the stacked
        # buffers are float32 (the others widen exactly), never the other way round
        names = [f"{p}experts.{e}.{n}_proj.weight" for e in range(E) for n in ("gate", "up", "down")]
        dt = torch.float32 if any(store.kept_dtype_of(n) == torch.float32 for n in names) else store.kept_dtype_of(names[0])
        self.w13 = torch.empty((E, 2 * I, H), dtype=dt, device=store.device)
        self.w2 = torch.empty((E, H, I), dtype=dt, device=store.device)
        for e in range(E):
            q = f"{p}experts.{e}."
            self.w13[e, :I].copy_(store.take(q + "gate_proj.weight"))
            self.w13[e, I:].copy_(store.take(q + "up_proj.weight"))
            self.w2[e].copy_(store.take(q + "down_proj.weight"))
        if S > 0:
            q = p + "shared_expert."
            g, u, d = (store.take(q + n + "_proj.weight") for n in ("gate", "up", "down"))
            sdt = torch.float32 if torch.float32 in (g.dtype, u.dtype, d.dtype) else g.dtype
            self.ws13 = torch.cat([g.to(sdt), u.to(sdt)], dim=0).unsqueeze(0).contiguous()
            self.ws2 = d.to(sdt).unsqueeze(0).contiguous()
            if self.shared_gate:
                self.w_shared_gate = store.get(p + "shared_expert_gate.weight")
        if store.run_dtype == torch.bfloat16 and H % 8 == 0 and self.w_router.dtype == torch.bfloat16:
            rows = [self.w_router]
            if self.w_shared_gate is not None:
                rows.append(self.w_shared_gate.to(torch.bfloat16).reshape(1, H))
            else:
                rows.append(torch.zeros((1, H), dtype=torch.bfloat16, device=store.device))
            self.w_router_packed = KT.pack_weights(torch.cat(rows, dim=0).contiguous(), False)
        # bfloat16 runs whose sizes give 16-byte rows keep the expert weights only in the packed layout
        # of the tensor-core kernel
        if store.run_dtype == torch.bfloat16 and H % 8 == 0 and I % 8 == 0 and KT.packable(self.w13) and KT.packable(self.w2):
            self.w13 = KT.pack_weights(self.w13, True)
            self.w2 = KT.pack_weights(self.w2, False)
        if self.ws13 is not None and store.run_dtype == torch.bfloat16 and H % 8 == 0 and S % 8 == 0 \
                and KT.packable(self.ws13) and KT.packable(self.ws2):
            self.ws13 = KT.pack_weights(self.ws13, True)
            self.ws2 = KT.pack_weights(self.ws2, False)

    def kernels(self) -> List[str]:
        names = ["moe", "elementwise"]
        dt = self.w13.dtype if self.w13 is not None else getattr(self, "run_dtype", torch.bfloat16)
        if dt == torch.bfloat16:
            names.append("gemm_tc")       # float32 runs never launch the tensor-core kernel
        return names

    def step_work(self, n_tokens, kv_tokens):
        E, k, H, I, S = self.n_experts, self.top_k, self.hidden, self.intermediate, self.shared_intermediate
        el = 4 if getattr(self, "run_dtype", None) == torch.float32 else 2
        touched = experts_touched(n_tokens, E, k)
        byt = el * (touched * 3 * H * I + 3 * H * S + (E + 1) * H)
        return {"moe": (byt, 2.0 * n_tokens * (k * 3 * H * I + 3 * H * S + (E + 1) * H))}

    _side_streams = {}

    @classmethod
    def _side_stream(cls, device):
        key = torch.device(device).index
        if key not in cls._side_streams:
            cls._side_streams[key] = torch.cuda.Stream(device=device)
        return cls._side_streams[key]

    EARLY_WEIGHTS = os.environ.get("TQ_EARLY_WEIGHTS", "1") not in ("", "0")
    EXACT_SHARED_ROWS = 2        # rows of the shared expert that the exact weight-stream kernel takes in one pass
    EXACT_FEW_ROWS = int(os.environ.get("TQ_EXACT_FEW_ROWS", "64"))      # steps of up to this many tokens take the exact kernels' weight-stream form

    def _product(self, x, w, out, layout, swiglu, token_tile, status=None, early=False):
        """Tensor cores for weights packed at load time (bfloat16, 16-byte rows), the exact CUDA-core
        kernel otherwise.  early: this is a down projection right behind its gate/up product in the stream: its
        weights and the layout were there before that product started, so it may stream weights while that runs."""
        if isinstance(w, KT.PackedWeights):
            return KT.gemm_tc(x, w, out, layout, token_tile, status=status, early_weights=early and self.EARLY_WEIGHTS)
        # the exact kernels: tiles of a few rows (decode steps) stream the weights; a group's tile holds at most the
        # step's tokens, and the one-group product (the shared expert) all of them
        rows = x.shape[0]
        few = rows <= self.EXACT_FEW_ROWS if layout is None else rows <= self.EXACT_FEW_ROWS * self.top_k
        return KM.grouped_gemm(x, w, out, layout, swiglu, few_rows=few)

    def _joint_launches(self, T: int, tile: int, act, dev) -> bool:
        """Whether the shared expert's two products ride in the routed experts' launches, their tiles ahead of the
        routed ones: steps of some hundred to about 1,500 tokens.  Either product alone fills the GPU with one
        persistent CTA per SM, so as launches of their own they run one after the other, and at these sizes each
        has only two to four rounds of tiles per CTA: its last round leaves SMs idle, which the other product's
        tiles fill when the same CTAs walk both.  (Measured on B200 at the A2.7B sizes, ms per prompt apart /
        together: 768 tokens 7.88 / 7.40, 1,024: 9.29 / 8.51, 1,536: 10.54 / 10.35, 2,048: 12.34 / 12.44, 8,192:
        44.9 / 45.8; at the 57B-A14B sizes 2,048 tokens: 16.5 / 16.8 over 8 layers.  Spreading the shared expert's
        tiles among the routed ones, a product bound by the tensor cores beside one bound by DRAM, is slower than
        either: both draw on the L2's bandwidth.  Giving each product a share of the SMs instead, as launches of
        their own on two streams, cost 25-60 %.)"""
        how = self.SHARED_IN_ROUTED_LAUNCH
        if (self.ws13 is None or tile < KT.PAIR_MIN_TILE or KT._NO_PAIRS or how == "0" or act != torch.bfloat16
                or not all(isinstance(w, KT.PackedWeights) for w in (self.w13, self.w2, self.ws13, self.ws2))):
            return False
        if how != "":
            return True
        return shared_rides_with_routed(T, self.shared_intermediate, KA_resident(dev))

    def forward(self, xn: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, H, k, dev = xn.shape[0], self.hidden, self.top_k, xn.device
        act = ctx.act_dtype
        # the shared expert does not depend on the routing: it runs on a second stream next to the routed experts
        # (its few CTAs would leave most of the GPU idle on their own), and in most steps it starts first, so that
        # the router's small kernels hide behind its weight stream
        y_shared = None
        side = None
        tile = KT.token_tile_for(T * k, self.n_experts) if isinstance(self.w13, KT.PackedWeights) else 0
        dual = self._joint_launches(T, tile, act, dev)
        if dual:
            tile = KT.TOKEN_TILES[-1]        # one width for both products; a tile's MMA is as wide as its own rows
        ids = torch.empty((T, k), dtype=torch.int32, device=dev)
        wts = torch.empty((T, k), dtype=torch.float32, device=dev)
        scale = torch.empty((T,), dtype=torch.float32, device=dev) if self.w_shared_gate is not None else None
        layout = KM.ExpertLayout(T * k, self.n_experts, tile or KM.TILE_ROWS, dev)
        x_rows = torch.empty((T * k, H), dtype=xn.dtype, device=dev)
        small = KM.router_small_pays(T, k, self.n_experts, H)
        # Decode steps whose pairs reach the number of experts (most experts are read: the routed products are several
        # times the shared expert's): the router first, alone on the GPU, then the shared expert beside the routed
        # ones with its down projection's K shared out.  With fewer pairs the shared expert starts first and the
        # router runs beside it.  (Measured on B200, tokens/s with the router first / with the shared expert first:
        # A2.7B sizes batch 8: 2,214 / 2,287, batch 16: 3,228 / 3,147; 57B-A14B sizes batch 1: 177 / 190, batch 8: 602 / 586.)
        shared_after = small and (T * k >= self.n_experts if self.SHARED_AFTER_ROUTER is None else self.SHARED_AFTER_ROUTER)

        def shared_expert():
            nonlocal y_shared, side
            S = self.shared_intermediate
            stile = KT.token_tile_for(T, 1) if isinstance(self.ws13, KT.PackedWeights) else 0
            main = torch.cuda.current_stream()
            side = self._side_stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                hs = torch.empty((T, S), dtype=act, device=dev)
                if not isinstance(self.ws13, KT.PackedWeights) and T > self.EXACT_SHARED_ROWS:
                    # unpacked weights (float32 runs, sizes the tensor-core kernel does not take) and more rows than
                    # one pass of the exact weight-stream kernel holds: the shared expert is a dense feed-forward, and
                    # the library's products serve it as they serve the dense layers
                    gu = linear(xn, self.ws13[0], out_dtype=torch.float32)
                    KE.silu_mul(gu, hs)
                    y_shared = linear(hs, self.ws2[0], out_dtype=torch.float32)
                    return
                self._product(xn, self.ws13, hs, None, True, stile, ctx.status)
                splits = 1
                if isinstance(self.ws2, KT.PackedWeights):
                    splits = shared_down_shares(T, self.n_experts, k, self.intermediate, S, H, stile, KA_resident(dev),
                                                shared_after, self.SHARED_DOWN_SPLIT_RATIO)
                y_shared = torch.empty((splits, T, H) if splits > 1 else (T, H), dtype=torch.float32, device=dev)
                if splits > 1:
                    KT.gemm_tc(hs, self.ws2, y_shared, None, stile, status=ctx.status, k_splits=splits, early_weights=self.EARLY_WEIGHTS)
                else:
                    self._product(hs, self.ws2, y_shared, None, False, stile, ctx.status, early=True)
            # hs and y_shared were allocated on the side stream; both live until this function returns,
            # after the main stream has joined the side stream again, and the side stream's next use
            # starts with a wait on the main stream: no cross-stream reuse hazard

        if self.ws13 is not None and not shared_after and not dual:
            shared_expert()
        if small:
            # few tokens (decoding): router, layout and the sorted copies of the rows in one launch
            KM.router_small(xn, self.w_router, self.w_shared_gate, k, self.norm_topk, ids, wts, scale, layout, x_rows)
        else:
            if self.w_router_packed is not None and T >= self.ROUTER_TC_MIN_TOKENS:
                # long steps (prompts): the logits of all tokens as one tensor-core product (bf16 x bf16 products
                # are exact in fp32 and the sum is fp32), then the selection kernel
                logits = torch.empty((T, self.n_experts + 1), dtype=torch.float32, device=dev)
                KT.gemm_tc(xn, self.w_router_packed, logits, None, KT.token_tile_for(T, 1), status=ctx.status)
                KM.router_select(logits, k, self.norm_topk, ids, wts, scale)
            else:
                KM.router_topk(xn, self.w_router, self.w_shared_gate, k, self.norm_topk, ids, wts, scale)
            KM.moe_align(ids, layout)
            KE.gather_rows(xn, layout.sorted_pair, k, x_rows)
        if self.ws13 is not None and shared_after and not dual:
            shared_expert()
        if ctx.debug is not None:
            # the tensors themselves: nothing below writes them, and inside a captured step a reference keeps their
            # memory from being reused, so that they hold every replay's choices
            ctx.debug.setdefault("router_ids", []).append(ids)
            ctx.debug.setdefault("router_weights", []).append(wts)
        h_rows = torch.empty((T * k, self.intermediate), dtype=act, device=dev)
        y_rows = torch.empty((T * k, H), dtype=torch.float32, device=dev)
        if dual:
            first = self.SHARED_IN_ROUTED_LAUNCH != "spread"
            hs = torch.empty((T, self.shared_intermediate), dtype=act, device=dev)
            y_shared = torch.empty((T, H), dtype=torch.float32, device=dev)
            KT.gemm_tc_dual(x_rows, self.w13, h_rows, layout, xn, self.ws13, hs, tile, ctx.status, first)
            KT.gemm_tc_dual(h_rows, self.w2, y_rows, layout, hs, self.ws2, y_shared, tile, ctx.status, first)
        else:
            self._product(x_rows, self.w13, h_rows, layout, True, tile, ctx.status)
            self._product(h_rows, self.w2, y_rows, layout, False, tile, ctx.status, early=True)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        y = torch.empty((T, H), dtype=torch.float32, device=dev)
        KM.moe_combine(y_rows, layout.row_of_pair, wts, y_shared, scale, y, k)
        return y


register_feed_forward("moe", MoEFeedForward)
