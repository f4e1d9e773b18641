"""More kinds of parts defined in a test and plugged into the framework without a change to its files:
a position encoding of its own (rotation angles that grow linearly with the pair index, handed to the
attention mixer as tables), one that is no rotation at all (queries and keys scaled by their position, through
the encoding's own apply()), and a feed-forward with routing of its own (every token goes to ONE of a few linear
maps, picked by the largest of its first features; built from the framework's layout, gather, grouped-product and
combine kernels).  A toy architecture made of them is registered, written as a random model folder, loaded by
its config.json and stepped whole, with a decoded tail, and in batches of unequal lengths, against a numpy
restatement in this file.  It is a test fixture, not anybody's model."""
import json
import os

import numpy as np
import pytest
import torch

from plain import qwen2_moe_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEAD = 16


def define_toy():
    import turboquant_cpp_b200 as tq
    from turboquant_cpp_b200.config import KeyReader
    from turboquant_cpp_b200.kernels import elementwise as KE, moe as KM
    from turboquant_cpp_b200.models import DecoderModel, Embedding, LMHead, ScheduleEntry
    from turboquant_cpp_b200.parts import (FeedForward, PositionEncoding, PreNormBlock, make_feed_forward, make_mixer,
                                           make_norm, make_position_encoding, register_feed_forward,
                                           register_position_encoding)
    from turboquant_cpp_b200.weights import WeightSpec

    class LinearAngles(PositionEncoding):
        """angle(pos, i) = pos * step * (i + 1): not the geometric schedule of the rotary part."""

        def __init__(self, head_dim, step, max_position):
            self.head_dim, self.step, self.max_position = head_dim, step, max_position
            self.cos = self.sin = None

        def prepare(self, device):
            i = torch.arange(1, self.head_dim // 2 + 1, dtype=torch.float64)
            ang = torch.arange(self.max_position, dtype=torch.float64)[:, None] * (self.step * i)[None, :]
            self.cos = torch.cos(ang).float().to(device).contiguous()
            self.sin = torch.sin(ang).float().to(device).contiguous()

        def tables(self):
            return self.cos, self.sin, "half"

    class ScaledByPosition(PositionEncoding):
        """Not a rotation: queries and keys are multiplied element by element by 1 + rate * pos * (i + 1) / head_dim.
        It has no tables, so the attention mixer calls apply() between the bias and the cache write."""

        def __init__(self, head_dim, rate):
            self.head_dim, self.rate = head_dim, rate

        def apply(self, q, k, positions):
            ramp = torch.arange(1, self.head_dim + 1, device=q.device, dtype=torch.float32) / self.head_dim
            f = (1.0 + self.rate * positions.float()[:, None, None] * ramp[None, None, :])
            q.mul_(f.to(q.dtype))
            if k is not None:
                k.mul_(f.to(k.dtype))

    class SwitchFeedForward(FeedForward):
        """y_t = W[e_t] x_t with e_t = argmax of the token's first n_maps features (ties to the lowest index)."""

        def __init__(self, prefix, hidden, n_maps):
            self.prefix, self.hidden, self.n_maps, self.w = prefix, hidden, n_maps, None

        def weight_specs(self):
            return [WeightSpec(f"{self.prefix}maps.{e}.weight", (self.hidden, self.hidden)) for e in range(self.n_maps)]

        def bind(self, store):
            self.w = torch.stack([store.take(f"{self.prefix}maps.{e}.weight") for e in range(self.n_maps)]).contiguous()

        def kernels(self):
            return ["moe", "elementwise"]

        def forward(self, xn, ctx):
            T, H = xn.shape
            ids = torch.argmax(xn[:, :self.n_maps].float(), dim=1, keepdim=True).to(torch.int32).contiguous()
            layout = KM.ExpertLayout(T, self.n_maps, KM.TILE_ROWS, xn.device)
            KM.moe_align(ids, layout)
            rows = KE.gather_rows(xn, layout.sorted_pair, 1, torch.empty((T, H), dtype=xn.dtype, device=xn.device))
            y_rows = KM.grouped_gemm(rows, self.w, torch.empty((T, H), dtype=torch.float32, device=xn.device), layout, False)
            ones = torch.ones((T, 1), dtype=torch.float32, device=xn.device)
            return KM.moe_combine(y_rows, layout.row_of_pair, ones, None, None,
                                  torch.empty((T, H), dtype=torch.float32, device=xn.device), 1)

    class ToyConfig:
        def __init__(self, raw, where):
            r = KeyReader(raw, where)
            self.hidden_size = r.integer("hidden_size", minimum=1)
            self.vocab_size = r.integer("vocab_size", minimum=1)
            self.max_position_embeddings = r.integer("max_position_embeddings", minimum=1)
            self.heads = r.integer("num_attention_heads", minimum=1)
            self.kv_heads = r.integer("num_key_value_heads", minimum=1)
            self.n_maps = r.integer("n_maps", minimum=1)
            self.n_layers = r.integer("num_hidden_layers", minimum=1)
            self.eps = r.real("rms_norm_eps", positive=True)
            self.step = r.real("angle_step", positive=True)
            self.window = r.integer("window", minimum=0)
            self.scaled_layers = r.int_list("scaled_layers", default=[])
            self.rate = r.real("scale_rate", default=0.01, positive=True)

        @classmethod
        def from_dict(cls, raw, where="config.json"):
            return cls(raw, where)

    class ToyModel(DecoderModel):
        def __init__(self, cfg, dtype):
            H = cfg.hidden_size
            pe = make_position_encoding("toy_linear_angles", head_dim=HEAD, step=cfg.step, max_position=cfg.max_position_embeddings)
            scaled = make_position_encoding("toy_scaled_by_position", head_dim=HEAD, rate=cfg.rate)
            blocks = []
            for l in range(cfg.n_layers):
                p = f"layers.{l}."
                blocks.append(PreNormBlock(
                    make_norm("rmsnorm", name=p + "n1.weight", size=H, eps=cfg.eps),
                    make_mixer("attention", prefix=p + "attn.", hidden=H, n_heads=cfg.heads, n_kv_heads=cfg.kv_heads,
                               head_dim=HEAD, qkv_bias=True, position=scaled if l in cfg.scaled_layers else pe,
                               window=cfg.window if l % 2 else 0),
                    make_norm("rmsnorm", name=p + "n2.weight", size=H, eps=cfg.eps),
                    make_feed_forward("toy_switch", prefix=p + "ff.", hidden=H, n_maps=cfg.n_maps)))
            super().__init__(cfg, dtype, Embedding("embed.weight", cfg.vocab_size, H), blocks,
                             [ScheduleEntry(l) for l in range(cfg.n_layers)],
                             make_norm("rmsnorm", name="final.weight", size=H, eps=cfg.eps),
                             LMHead("head.weight", cfg.vocab_size, H))

    register_position_encoding("toy_linear_angles", LinearAngles, replace=True)
    register_position_encoding("toy_scaled_by_position", ScaledByPosition, replace=True)
    register_feed_forward("toy_switch", SwitchFeedForward, replace=True)
    tq.register_architecture("ToySwitchLM", ToyConfig, ToyModel, replace=True)


TOY_CONFIG = {"architectures": ["ToySwitchLM"], "hidden_size": 40, "vocab_size": 83, "max_position_embeddings": 200,
              "num_attention_heads": 4, "num_key_value_heads": 2, "n_maps": 5, "num_hidden_layers": 3,
              "rms_norm_eps": 1e-5, "angle_step": 0.013, "window": 24, "scaled_layers": [1], "scale_rate": 0.01}


def rotate(x, positions, step):
    T, nh, hd = x.shape
    ang = positions.astype(np.float64)[:, None] * (step * np.arange(1, hd // 2 + 1))[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :hd // 2], x[..., hd // 2:]
    return np.concatenate([a * cos - b * sin, a * sin + b * cos], axis=-1)


def toy_plain_forward(w, cfg, tokens, margins=None):
    """Whole-sequence numpy restatement.  margins: list that receives, per layer, each token's gap between its
    largest and second largest routing feature."""
    nh, nkv, E = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["n_maps"]
    T = len(tokens)
    pos = np.arange(T)
    x = w["embed.weight"][np.asarray(tokens)]
    for l in range(cfg["num_hidden_layers"]):
        p = f"layers.{l}."
        xn = P.rmsnorm(x, w[p + "n1.weight"], cfg["rms_norm_eps"])
        a = p + "attn."
        if l in cfg.get("scaled_layers", []):
            f = 1.0 + cfg["scale_rate"] * pos[:, None, None] * (np.arange(1, HEAD + 1) / HEAD)[None, None, :]
            encode = lambda x: x * f
        else:
            encode = lambda x: rotate(x, pos, cfg["angle_step"])
        q = encode((P.linear(xn, w[a + "q_proj.weight"]) + w[a + "q_proj.bias"]).reshape(T, nh, HEAD))
        k = encode((P.linear(xn, w[a + "k_proj.weight"]) + w[a + "k_proj.bias"]).reshape(T, nkv, HEAD))
        v = (P.linear(xn, w[a + "v_proj.weight"]) + w[a + "v_proj.bias"]).reshape(T, nkv, HEAD)
        x = x + P.linear(P.attention(q, k, v, cfg["window"] if l % 2 else 0), w[a + "o_proj.weight"])
        xn = P.rmsnorm(x, w[p + "n2.weight"], cfg["rms_norm_eps"])
        e = np.argmax(xn[:, :E], axis=1)
        if margins is not None:
            s = np.sort(xn[:, :E], axis=1)
            margins.append(s[:, -1] - s[:, -2])
        x = x + np.stack([w[f"{p}ff.maps.{e[t]}.weight"] @ xn[t] for t in range(T)])
    return P.linear(P.rmsnorm(x, w["final.weight"], cfg["rms_norm_eps"]), w["head.weight"])


def test_toy_position_encoding_and_routed_feed_forward_plug_in(tmp_path):
    import turboquant_cpp_b200 as tq
    from replay_util import batched, run_schedule, whole, with_tail
    define_toy()
    folder = str(tmp_path / "toy_switch")
    tq.write_random_folder(folder, TOY_CONFIG, seed=11, std=0.2)
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToySwitchLM"]
    model = tq.load_model(folder, "float32", DEV)                       # the class is chosen by config.json
    assert type(model).__name__ == "ToyModel" and len(model.schedule) == 3
    eng = tq.Engine(model, max_tokens=1024, record_routing=True)
    assert len(eng.cache.groups) == 2                                   # full and windowed layers keep their own pages
    w = P.read_safetensors(os.path.join(folder, "model.safetensors"))
    rng = np.random.default_rng(12)
    reqs = {"a": rng.integers(0, 83, size=50).tolist(), "b": rng.integers(0, 83, size=120).tolist(),
            "c": rng.integers(0, 83, size=9).tolist()}
    refs = {}
    for r, t in reqs.items():
        margins = []
        refs[r] = toy_plain_forward(w, TOY_CONFIG, t, margins)
        assert min(m.min() for m in margins) > 1e-4, "a routing near-tie: pick another seed"

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
    for _ in range(2):                                                    # twice: slots are used again
        logits, _ = run_schedule(eng, *batched(reqs, {"a": 17, "b": 70, "c": 9}))
        check(logits, "batched")
        assert all(sorted(logits[r]) == list(range(len(reqs[r]))) for r in reqs)
    eng.cache.book.check_invariants()
    tq.config.unregister_architecture("ToySwitchLM")
