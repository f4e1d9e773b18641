"""Each part alone against the plain function for the same part, and a toy architecture defined
here — a mixer with per-sequence state of its own, a block named twice in the layer schedule, an
entry that reads another entry's cache — registered, built, loaded and stepped without a change
to the framework's files."""
import json
import math
import os
import types

import numpy as np
import pytest
import torch

from plain import qwen2_moe_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def store_for(part, seed, dtype=torch.float32):
    from turboquant_cpp_b200.weights import RandomSource, WeightStore
    specs = part.weight_specs()
    return WeightStore(RandomSource(specs, seed, std=0.1), specs, DEV, dtype), specs


def plain_weights(store, specs):
    return {s.name: store.get(s.name).double().cpu().numpy() for s in specs}


def context_for(q_lens, starts, act_dtype, cache):
    """A StepContext and the device page tables for sequences that already hold `starts` tokens."""
    from turboquant_cpp_b200.parts import StepContext
    seqs = []
    for s in starts:
        seq = cache.open()
        if s:
            cache.reserve([seq], [s])
            cache.commit([seq], [s])
        seqs.append(seq)
    cache.reserve(seqs, q_lens)
    B, T = len(q_lens), sum(q_lens)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    seq_of = np.repeat(np.arange(B), q_lens)
    pos = np.arange(T) - cu[:-1][seq_of] + np.asarray(starts)[seq_of]
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    ctx = StepContext(n_tokens=T, n_seqs=B, tokens=i32(np.zeros(T)), positions=i32(pos), seq_of_token=i32(seq_of),
                      cu_seqlens=i32(cu), seq_start=i32(starts), slots=i32([s.slot for s in seqs]),
                      want_rows=i32([]), n_want=0, max_q_len=max(q_lens), max_kv_len=max(a + b for a, b in zip(starts, q_lens)),
                      act_dtype=act_dtype, device=torch.device(DEV), host_q_lens=list(q_lens),
                      host_slots=[s.slot for s in seqs])
    tables = [i32(t) for t in cache.page_tables(seqs)]
    return ctx, tables, seqs


def close(got, want, tol):
    got = got.detach().double().cpu().numpy()
    err = np.abs(got - want).max() / max(1e-30, np.abs(want).max())
    assert err < tol, f"relative error {err:.3e} exceeds {tol:.1e}"


def test_norm_part():
    from turboquant_cpp_b200.parts import make_norm
    n = make_norm("rmsnorm", name="n.weight", size=70, eps=1e-4)
    store, specs = store_for(n, 1)
    n.bind(store)
    w = plain_weights(store, specs)["n.weight"]
    x = torch.randn(9, 70, device=DEV)
    y = torch.randn(9, 70, device=DEV)
    close(n.forward(x, torch.float32), P.rmsnorm(x.double().cpu().numpy(), w, 1e-4), 3e-6)
    xs = (x.double() + y.double()).cpu().numpy()
    close(n.add_forward(x, y, torch.float32), P.rmsnorm(xs, w, 1e-4), 3e-6)
    close(x, xs, 1e-6)


@pytest.mark.parametrize("pairing", ["half", "interleaved"])
def test_rotary_part_tables(pairing):
    from turboquant_cpp_b200.parts import make_position_encoding
    r = make_position_encoding("rotary", head_dim=48, theta=777.0, max_position=300, pairing=pairing)
    r.prepare(DEV)
    cos, sin, pr = r.tables()
    assert pr == pairing and cos.shape == (300, 24) and cos.dtype == torch.float32
    i = np.arange(24)
    ang = np.arange(300)[:, None] / np.power(777.0, 2 * i / 48)[None, :]
    close(cos, np.cos(ang), 1e-7)
    close(sin, np.sin(ang), 1e-7)


@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 4, 16, 0), (6, 2, 32, 5), (5, 1, 48, 0)])
def test_attention_mixer_alone(nh, nkv, hd, window):
    """Two sequences, one fresh and one that already holds 70 tokens written by an earlier call."""
    from turboquant_cpp_b200.cache import PagedCache
    from turboquant_cpp_b200.parts import make_mixer, make_position_encoding
    H = 72
    rot = make_position_encoding("rotary", head_dim=hd, theta=5000.0, max_position=256, pairing="half")
    mix = make_mixer("attention", prefix="model.layers.0.self_attn.", hidden=H, n_heads=nh, n_kv_heads=nkv,
                     head_dim=hd, qkv_bias=True, window=window, position=rot)
    store, specs = store_for(mix, 2)
    w = plain_weights(store, specs)
    mix.bind(store)
    cache = PagedCache([mix.cache_need()], [None], [None], 1024, torch.float32, DEV)
    m = types.SimpleNamespace(w=w, nh=nh, nkv=nkv, hd=hd, theta=5000.0, layer_window=lambda l: window)
    x_old = torch.randn(70, H, device=DEV)
    ctx, tables, seqs = context_for([70], [0], torch.float32, cache)
    y_old = mix.forward(x_old, ctx, cache.layer_caches(tables)[0])
    cache.commit(seqs, [70])
    close(y_old, P.attention_mixer(m, 0, x_old.double().cpu().numpy(), np.arange(70)), 5e-6)
    # the same sequence goes on by 3 tokens, next to a new sequence of 9
    x_new = torch.randn(12, H, device=DEV)
    seq2 = cache.open()
    cache.reserve([seqs[0], seq2], [3, 9])
    ctx, tables = context_from_seqs([seqs[0], seq2], [3, 9], torch.float32, cache)
    y = mix.forward(x_new, ctx, cache.layer_caches(tables)[0])
    full = np.concatenate([x_old.double().cpu().numpy(), x_new[:3].double().cpu().numpy()])
    close(y[:3], P.attention_mixer(m, 0, full, np.arange(73))[70:], 5e-6)
    close(y[3:], P.attention_mixer(m, 0, x_new[3:].double().cpu().numpy(), np.arange(9)), 5e-6)


def context_from_seqs(seqs, q_lens, act_dtype, cache):
    from turboquant_cpp_b200.parts import StepContext
    starts = [s.length for s in seqs]
    B, T = len(q_lens), sum(q_lens)
    cu = np.concatenate([[0], np.cumsum(q_lens)])
    seq_of = np.repeat(np.arange(B), q_lens)
    pos = np.arange(T) - cu[:-1][seq_of] + np.asarray(starts)[seq_of]
    i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
    ctx = StepContext(n_tokens=T, n_seqs=B, tokens=i32(np.zeros(T)), positions=i32(pos), seq_of_token=i32(seq_of),
                      cu_seqlens=i32(cu), seq_start=i32(starts), slots=i32([s.slot for s in seqs]),
                      want_rows=i32([]), n_want=0, max_q_len=max(q_lens), max_kv_len=max(a + b for a, b in zip(starts, q_lens)),
                      act_dtype=act_dtype, device=torch.device(DEV), host_q_lens=list(q_lens),
                      host_slots=[s.slot for s in seqs])
    return ctx, [i32(t) for t in cache.page_tables(seqs)]


def test_dense_feed_forward_alone():
    from turboquant_cpp_b200.parts import make_feed_forward
    ff = make_feed_forward("swiglu", prefix="model.layers.0.mlp.", hidden=50, intermediate=70)
    store, specs = store_for(ff, 3)
    w = plain_weights(store, specs)
    ff.bind(store)
    x = torch.randn(11, 50, device=DEV)
    ctx = types.SimpleNamespace(act_dtype=torch.float32, debug=None, status=None)
    m = types.SimpleNamespace(w=w)
    close(ff.forward(x, ctx), P.dense_feed_forward(m, 0, x.double().cpu().numpy()), 5e-6)


@pytest.mark.parametrize("E,k,I,S,norm", [(8, 2, 32, 64, False), (6, 3, 48, 128, True), (5, 1, 40, 0, False)])
def test_moe_feed_forward_alone(E, k, I, S, norm):
    from turboquant_cpp_b200.parts import make_feed_forward
    H = 56
    ff = make_feed_forward("moe", prefix="model.layers.0.mlp.", hidden=H, n_experts=E, top_k=k, intermediate=I,
                           norm_topk=norm, shared_intermediate=S)
    store, specs = store_for(ff, 4)
    w = plain_weights(store, specs)
    ff.bind(store)
    x = torch.randn(40, H, device=DEV)
    ctx = types.SimpleNamespace(act_dtype=torch.float32, debug={}, status=None)
    y = ff.forward(x, ctx)
    m = types.SimpleNamespace(w=w, k=k, norm_topk=norm, cfg={"shared_expert_intermediate_size": S})
    rec = {}
    want = P.moe_feed_forward(m, 0, x.double().cpu().numpy(), record=rec)
    assert rec["margin"][0].min() > 1e-4
    assert np.array_equal(ctx.debug["router_ids"][0].cpu().numpy(), rec["ids"][0])
    close(y, want, 5e-6)


# ------------------------------------------------------------------------------------------------
# a toy architecture, defined here
# ------------------------------------------------------------------------------------------------
def define_toy():
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.config import KeyReader
    from turboquant_cpp_b200.models import DecoderModel, Embedding, LMHead, ScheduleEntry
    from turboquant_cpp_b200.parts import (Mixer, PreNormBlock, StateNeed, make_feed_forward, make_mixer, make_norm,
                                           make_position_encoding, register_mixer)
    from turboquant_cpp_b200.weights import WeightSpec

    class RunningMeanMixer(Mixer):
        """y_t = W · mean(x_0 … x_t): the state of a sequence is the running sum and the count."""

        def __init__(self, prefix, hidden):
            self.prefix, self.hidden, self.w = prefix, hidden, None

        def weight_specs(self):
            return [WeightSpec(self.prefix + "mean_proj.weight", (self.hidden, self.hidden))]

        def bind(self, store):
            self.w = store.get(self.prefix + "mean_proj.weight").float()

        def state_need(self):
            return StateNeed((self.hidden + 1,), torch.float32)

        def forward(self, xn, ctx, cache):
            # everything that changes from step to step comes from device tensors of the context (slots,
            # seq_of_token, cu_seqlens), so a decode step of this mixer can be recorded into a CUDA graph; every
            # token updates its sequence's state exactly once
            H = self.hidden
            seq = ctx.seq_of_token.long()
            slots = ctx.slots.long()
            x = xn.float()
            run = torch.cumsum(x, dim=0)                                   # over the whole step …
            first = ctx.cu_seqlens[:-1].long()                             # … minus what came before each sequence
            before = torch.cat([torch.zeros((1, H), device=x.device), run])[first]
            st = cache.state[slots]                                        # [B, H + 1]: running sum, count
            sums = run - before[seq] + st[seq, :H]
            place = torch.arange(x.shape[0], device=x.device) - first[seq] + 1
            counts = st[seq, H] + place.float()
            last = ctx.cu_seqlens[1:].long() - 1
            cache.state[slots] = torch.cat([sums[last], counts[last, None]], dim=1)
            return (sums / counts[:, None]) @ self.w.t()

    class ToyConfig:
        def __init__(self, raw, where):
            r = KeyReader(raw, where)
            self.hidden_size = r.integer("hidden_size", minimum=1)
            self.vocab_size = r.integer("vocab_size", minimum=1)
            self.max_position_embeddings = r.integer("max_position_embeddings", minimum=1)
            self.intermediate_size = r.integer("intermediate_size", minimum=1)
            self.heads = r.integer("num_attention_heads", minimum=1)
            self.eps = r.real("rms_norm_eps", positive=True)
            self.theta = r.real("rope_theta", positive=True)
            self.layer_order = r.int_list("layer_order")
            self.share_last_cache = r.boolean("share_last_cache", default=False)

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(raw, where)

    class ToyModel(DecoderModel):
        def __init__(self, cfg, dtype):
            H = cfg.hidden_size
            rot = make_position_encoding("rotary", head_dim=16, theta=cfg.theta, max_position=cfg.max_position_embeddings)

            def block(i, mixer):
                p = f"layers.{i}."
                return PreNormBlock(make_norm("rmsnorm", name=p + "n1.weight", size=H, eps=cfg.eps), mixer,
                                    make_norm("rmsnorm", name=p + "n2.weight", size=H, eps=cfg.eps),
                                    make_feed_forward("swiglu", prefix=p + "mlp.", hidden=H, intermediate=cfg.intermediate_size))
            blocks = [block(0, make_mixer("toy_running_mean", prefix="layers.0.mix.", hidden=H)),
                      block(1, make_mixer("attention", prefix="layers.1.attn.", hidden=H, n_heads=cfg.heads,
                                          n_kv_heads=1, head_dim=16, qkv_bias=False, position=rot))]
            schedule, last_attn = [], None
            for j, b in enumerate(cfg.layer_order):
                share = cfg.share_last_cache and b == 1 and last_attn is not None and j == len(cfg.layer_order) - 1
                schedule.append(ScheduleEntry(b, cache_of=last_attn if share else None))
                if b == 1 and not share:
                    last_attn = j
            super().__init__(cfg, dtype, Embedding("embed.weight", cfg.vocab_size, H), blocks, schedule,
                             make_norm("rmsnorm", name="final.weight", size=H, eps=cfg.eps),
                             LMHead("embed.weight", cfg.vocab_size, H))

    register_mixer("toy_running_mean", RunningMeanMixer, replace=True)
    tq.register_architecture("ToyStatefulLM", ToyConfig, ToyModel, replace=True)
    return ToyModel


TOY_CONFIG = {"architectures": ["ToyStatefulLM"], "hidden_size": 48, "vocab_size": 97, "max_position_embeddings": 160,
              "intermediate_size": 40, "num_attention_heads": 3, "rms_norm_eps": 1e-5, "rope_theta": 1000.0,
              "layer_order": [0, 1, 0, 1], "share_last_cache": True}


def toy_plain_forward(w, cfg, tokens):
    """Whole-sequence numpy restatement of the toy model."""
    H, nh, hd = cfg["hidden_size"], cfg["num_attention_heads"], 16
    T = len(tokens)
    pos = np.arange(T)
    x = w["embed.weight"][np.asarray(tokens)]
    kv_of = {}
    order = cfg["layer_order"]
    for j, b in enumerate(order):
        p = f"layers.{b}."
        xn = P.rmsnorm(x, w[p + "n1.weight"], cfg["rms_norm_eps"])
        if b == 0:
            mean = np.cumsum(xn, axis=0) / np.arange(1, T + 1)[:, None]
            y = mean @ w["layers.0.mix.mean_proj.weight"].T
        else:
            a = "layers.1.attn."
            q = P.rotary(P.linear(xn, w[a + "q_proj.weight"]).reshape(T, nh, hd), pos, cfg["rope_theta"])
            shared = cfg["share_last_cache"] and j == len(order) - 1 and 1 in order[:j]
            if shared:
                k, v = kv_of[max(i for i in range(j) if order[i] == 1)]
            else:
                k = P.rotary(P.linear(xn, w[a + "k_proj.weight"]).reshape(T, 1, hd), pos, cfg["rope_theta"])
                v = P.linear(xn, w[a + "v_proj.weight"]).reshape(T, 1, hd)
                kv_of[j] = (k, v)
            y = P.linear(P.attention(q, k, v, 0), w[a + "o_proj.weight"])
        x = x + y
        xn = P.rmsnorm(x, w[p + "n2.weight"], cfg["rms_norm_eps"])
        x = x + P.swiglu(xn, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.linear(P.rmsnorm(x, w["final.weight"], cfg["rms_norm_eps"]), w["embed.weight"])


def test_toy_architecture_registers_builds_loads_and_steps(tmp_path):
    import turboquant_cpp_b200 as tq
    from replay_util import batched, run_schedule, whole, with_tail
    define_toy()
    folder = str(tmp_path / "toy")
    tq.write_random_folder(folder, TOY_CONFIG, seed=5, std=0.1)
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyStatefulLM"]
    model = tq.load_model(folder, "float32", DEV)                       # the class is chosen by config.json
    assert type(model).__name__ == "ToyModel" and len(model.schedule) == 4
    assert model.schedule[3].cache_of == 1 and model.schedule[2].block == 0
    eng = tq.Engine(model, max_tokens=1024, record_routing=True)
    assert eng.graphs is not None and not eng.can_step_ahead     # decode steps run as CUDA graphs; with state of its own
    #                                                              no step is launched before the one before is kept
    assert len(eng.cache.groups) == 1 and eng.cache.kv[3] is eng.cache.kv[1] and eng.cache.kv[0] is None
    assert eng.cache.state[0] is not None and eng.cache.state[2] is not None and eng.cache.state[0] is not eng.cache.state[2]
    w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(6)
    reqs = {"a": rng.integers(0, 97, size=45).tolist(), "b": rng.integers(0, 97, size=100).tolist(),
            "c": rng.integers(0, 97, size=7).tolist()}
    refs = {r: toy_plain_forward(w, TOY_CONFIG, t) for r, t in reqs.items()}

    def check(logits, what):
        for r, ref in refs.items():
            if r in logits:
                for p, row in logits[r].items():
                    err = np.abs(row - ref[p]).max() / np.abs(ref).max()
                    assert err < 2e-5, f"{what} {r} position {p}: {err:.2e}"
    for r, t in reqs.items():
        logits, _ = run_schedule(eng, *whole(r, t))
        check(logits, "whole")
        logits, _ = run_schedule(eng, *with_tail(r, t, 32))
        check(logits, "tail")
    for _ in range(2):                                                    # twice: slots and their state are used again
        logits, _ = run_schedule(eng, *batched(reqs, {"a": 13, "b": 68, "c": 7}))
        check(logits, "batched")
        assert all(sorted(logits[r]) == list(range(len(reqs[r]))) for r in reqs)
    eng.cache.book.check_invariants()
    assert eng.graphs.graphs, "no decode step was captured"
    # a part that says it cannot be captured keeps the model's decode steps out of graphs, nothing else changes
    model.blocks[0].mixer.capturable = lambda: False
    eager = tq.Engine(model, max_tokens=1024)
    assert eager.graphs is None
    logits, _ = run_schedule(eager, *with_tail("b", reqs["b"], 8))
    check(logits, "uncaptured tail")
    tq.config.unregister_architecture("ToyStatefulLM")


def test_block_embedding_and_head_alone():
    """A whole pre-norm block (norm, attention, add, norm, experts, add), the embedding and the LM head."""
    from turboquant_cpp_b200.cache import PagedCache
    from turboquant_cpp_b200.models import Embedding, LMHead
    from turboquant_cpp_b200.parts import (PreNormBlock, make_feed_forward, make_mixer, make_norm,
                                           make_position_encoding)
    H, nh, nkv, hd, E, k, I, S, V = 48, 3, 1, 16, 4, 2, 24, 40, 50
    rot = make_position_encoding("rotary", head_dim=hd, theta=300.0, max_position=128, pairing="half")
    p = "model.layers.0."
    blk = PreNormBlock(
        make_norm("rmsnorm", name=p + "input_layernorm.weight", size=H, eps=1e-5),
        make_mixer("attention", prefix=p + "self_attn.", hidden=H, n_heads=nh, n_kv_heads=nkv, head_dim=hd,
                   qkv_bias=True, window=0, position=rot),
        make_norm("rmsnorm", name=p + "post_attention_layernorm.weight", size=H, eps=1e-5),
        make_feed_forward("moe", prefix=p + "mlp.", hidden=H, n_experts=E, top_k=k, intermediate=I, norm_topk=True,
                          shared_intermediate=S))
    emb, head = Embedding("model.embed_tokens.weight", V, H), LMHead("lm_head.weight", V, H)
    from turboquant_cpp_b200.weights import RandomSource, WeightStore
    specs = blk.weight_specs() + emb.weight_specs() + head.weight_specs()
    store = WeightStore(RandomSource(specs, 9, std=0.1), specs, DEV, torch.float32)
    w = plain_weights(store, specs)
    for part in (blk, emb, head):
        part.bind(store)
    toks = np.random.default_rng(0).integers(0, V, size=20)
    x = emb.forward(torch.tensor(toks, dtype=torch.int32, device=DEV))
    close(x, P.embedding(w["model.embed_tokens.weight"], toks), 1e-7)
    cache = PagedCache([blk.mixer.cache_need()], [None], [None], 256, torch.float32, DEV)
    ctx, tables, seqs = context_for([20], [0], torch.float32, cache)
    x0 = x.double().cpu().numpy()
    xr, pending = blk.forward(x, None, ctx, cache.layer_caches(tables)[0])
    m = types.SimpleNamespace(w=w, L=1, H=H, nh=nh, nkv=nkv, hd=hd, eps=1e-5, theta=300.0, E=E, k=k, norm_topk=True,
                              cfg={"shared_expert_intermediate_size": S}, layer_is_sparse=lambda l: True,
                              layer_window=lambda l: 0)
    want = P.block(m, 0, x0, np.arange(20))
    close(xr + pending, want, 1e-5)
    close(head.forward(xr + pending), P.linear((xr + pending).double().cpu().numpy(), w["lm_head.weight"]), 1e-5)
