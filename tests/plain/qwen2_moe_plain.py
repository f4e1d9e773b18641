"""Plain, slow implementation of the Qwen2 MoE decoder, for tests only.

Whole sequences, no cache, no batching, numpy float64, one function for each
part.  It shares no code with the product path: it has its own reader of
config.json and of safetensors files.  Each function is written from the
reference's formulas and cites where the reference computes the same thing
(paths are relative to the reference's project root).  The reference's model
code compiles on the CPU; tests/golden/ holds the outputs of one run of it on
a tiny random model and the script that made them, and test_golden.py
compares this file with those outputs once.

Where this architecture needs something the reference does not have, the
function says so:
  * rotary pairing "half" (x[i], x[i+hd/2]) — the layout of safetensors
    checkpoints; the reference rotates interleaved pairs;
  * norm_topk_prob=false — the reference always renormalises;
  * a per-layer sliding window for this family — the reference has it for
    Gemma only;
  * exact exp in the experts' SiLU and the shared gate's sigmoid — the
    reference uses a fast approximation there (src/engine/tq_moe.c:42-48).

``act_round`` emulates a run that stores activations in bfloat16: it is
applied at the places where the engine's bfloat16 path writes an activation
tensor, and is the identity for float32 comparisons.
"""
from __future__ import annotations

import json
import os
import struct
from typing import Callable, Dict, List, Optional, Sequence

import numpy as np

Round = Callable[[np.ndarray], np.ndarray]


def no_round(a: np.ndarray) -> np.ndarray:
    return a


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    f = np.asarray(a, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


# ------------------------------------------------------------------------------------
# reading a model folder (own reader; layout as in src/engine/tq_model.c:185-305)
# ------------------------------------------------------------------------------------
def _widen(raw, dt: str, name: str, shape) -> np.ndarray:
    if dt == "BF16":       # widen by a 16-bit shift, src/engine/tq_model.c:367-412
        a = (np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
    elif dt == "F32":
        a = np.frombuffer(raw, dtype=np.float32)
    elif dt == "F16":
        a = np.frombuffer(raw, dtype=np.float16)
    elif dt == "I32":
        a = np.frombuffer(raw, dtype=np.int32)
    else:
        raise ValueError(f"plain reader: dtype {dt} of '{name}' not handled")
    return a.astype(np.float64 if dt != "I32" else np.int64).reshape(shape)


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as f:
        blob = f.read()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    data = blob[8 + hlen:]
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        out[name] = _widen(data[b:e], info["dtype"], name, info["shape"])
    return out


class TensorsOnDemand:
    """The tensors of a folder's files, each widened to float64 when it is asked for and not kept (small ones
    are): for models whose tensors do not fit the host's memory as float64 all at once."""
    KEEP_BELOW = 1 << 20          # elements

    def __init__(self, paths: Sequence[str]):
        self.where, self.kept, self.maps = {}, {}, []
        for path in paths:
            mm = np.memmap(path, dtype=np.uint8, mode="r")
            (hlen,) = struct.unpack("<Q", bytes(mm[:8]))
            header = json.loads(bytes(mm[8:8 + hlen]).decode("utf-8"))
            self.maps.append(mm)
            for name, info in header.items():
                if name != "__metadata__":
                    b, e = info["data_offsets"]
                    self.where[name] = (mm, 8 + hlen + b, 8 + hlen + e, info["dtype"], info["shape"])

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def __getitem__(self, name: str) -> np.ndarray:
        if name in self.kept:
            return self.kept[name]
        mm, b, e, dt, shape = self.where[name]
        a = _widen(mm[b:e], dt, name, shape)
        if a.size < self.KEEP_BELOW:
            self.kept[name] = a
        return a

    def get(self, name: str, default=None):
        return self[name] if name in self.where else default


class PlainModel:
    """config.json (as a dict) and the tensors of a folder, by name.  on_demand: tensors are widened when they
    are used instead of all at once (for layers of real models' widths)."""

    def __init__(self, folder: str, on_demand: bool = False):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        files = [os.path.join(folder, n) for n in sorted(os.listdir(folder)) if n.endswith(".safetensors")]
        if on_demand:
            self.w = TensorsOnDemand(files)
        else:
            self.w: Dict[str, np.ndarray] = {}
            for path in files:
                self.w.update(read_safetensors(path))
        c = self.cfg
        self.L = c["num_hidden_layers"]
        self.H = c["hidden_size"]
        self.nh = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nh)
        self.hd = c.get("head_dim", self.H // self.nh)
        self.eps = c["rms_norm_eps"]
        self.theta = c["rope_theta"]
        self.E = c["num_experts"]
        self.k = c["num_experts_per_tok"]
        self.norm_topk = c.get("norm_topk_prob", False)
        self.tied = c.get("tie_word_embeddings", False)

    def layer_is_sparse(self, l: int) -> bool:
        c = self.cfg
        return (l not in c.get("mlp_only_layers", []) and self.E > 0
                and (l + 1) % c.get("decoder_sparse_step", 1) == 0)

    def layer_window(self, l: int) -> int:
        c = self.cfg
        if c.get("use_sliding_window", False) and l >= c.get("max_window_layers", self.L):
            return c["sliding_window"]
        return 0


# ------------------------------------------------------------------------------------
# parts
# ------------------------------------------------------------------------------------
def embedding(table: np.ndarray, tokens: Sequence[int]) -> np.ndarray:
    """x = table[token], no scaling for this family (src/engine/tq_transformer.c:2298-2329;
    the sqrt(H) scale at :2332-2337 is Gemma's)."""
    return table[np.asarray(tokens, dtype=np.int64)].copy()


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """ss = sum(x^2)/n + eps; y = x * (1/sqrt(ss)) * w, the weight used as it is
    (src/engine/tq_ops.c:1373-1410, scalar branch :1400-1408)."""
    ss = (x * x).sum(axis=-1, keepdims=True) / x.shape[-1] + eps
    return x * (1.0 / np.sqrt(ss)) * weight


def linear(x: np.ndarray, w: np.ndarray, b: Optional[np.ndarray] = None) -> np.ndarray:
    """out[i] = sum_j W[i,j] x[j] for row-major W [out, in] (src/engine/tq_ops.c:270-277);
    the bias is added after the product (src/engine/tq_transformer.c:1044-1047, 1086-1093)."""
    y = x @ w.T
    return y if b is None else y + b


def rotary(x: np.ndarray, positions: np.ndarray, theta: float, pairing: str = "half") -> np.ndarray:
    """x: [T, heads, hd].  freq_i = theta^(-2i/hd), angle = pos*freq_i,
    (a, b) <- (a cos - b sin, a sin + b cos) (src/engine/tq_ops.c:1418-1448).
    The reference pairs (x[2i], x[2i+1]) ("interleaved"); safetensors checkpoints of this
    family pair (x[i], x[i+hd/2]) ("half"), which is this library's default."""
    T, nh, hd = x.shape
    i = np.arange(hd // 2, dtype=np.float64)
    freq = 1.0 / np.power(float(theta), 2.0 * i / hd)
    ang = positions.astype(np.float64)[:, None] * freq[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = np.empty_like(x)
    if pairing == "interleaved":
        a, b = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = a * cos - b * sin
        out[..., 1::2] = a * sin + b * cos
    elif pairing == "half":
        a, b = x[..., :hd // 2], x[..., hd // 2:]
        out[..., :hd // 2] = a * cos - b * sin
        out[..., hd // 2:] = a * sin + b * cos
    else:
        raise ValueError(pairing)
    return out


def softmax(s: np.ndarray) -> np.ndarray:
    """max-subtract, exp, normalise (src/engine/tq_ops.c:1496-1519)."""
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int) -> np.ndarray:
    """q [T, nh, hd], k/v [T, nkv, hd] of one whole sequence -> [T, nh*hd].
    Head h reads KV head h // (nh/nkv) (src/engine/tq_transformer.c:1675-1680); scores are
    q.k / sqrt(hd) (:1633, :1909-1936) over positions start..t, softmax (:1960), weighted sum
    of V (:2183-2191).  start = max(0, t+1-window) on a windowed layer, as the reference's
    Gemma branch does (:1646-1654); 0 otherwise."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    out = np.zeros((T, nh, hd))
    scale = 1.0 / np.sqrt(hd)
    t = np.arange(T)
    start = np.maximum(0, t + 1 - window) if window > 0 else np.zeros(T, dtype=np.int64)
    seen = (t[None, :] <= t[:, None]) & (t[None, :] >= start[:, None])        # [query, key]
    for h in range(nh):
        g = h // (nh // nkv)
        s = np.where(seen, (q[:, h] @ k[:, g].T) * scale, -np.inf)          # one head, all queries at once
        out[:, h] = softmax(s) @ v[:, g]
    return out.reshape(T, nh * hd)


def silu(x: np.ndarray) -> np.ndarray:
    """x / (1 + exp(-x)) (src/engine/tq_ops.c:1454-1478)."""
    return x / (1.0 + np.exp(-x))


# exp used by the experts' SiLU and the shared gate's sigmoid.  The library's formula is the exact
# exponential; tests/test_golden.py swaps in the reference's fast approximation
# (src/engine/tq_moe.c:42-48) to compare with the reference's own output.
MOE_EXP = np.exp


def swiglu(x: np.ndarray, wg: np.ndarray, wu: np.ndarray, wd: np.ndarray, rnd: Round = no_round, exp=np.exp) -> np.ndarray:
    """down(silu(gate x) * (up x)) (dense: src/engine/tq_transformer.c:2771-2806;
    experts: src/engine/tq_moe.c:975-999, with exact exp here)."""
    g = linear(x, wg)
    h = rnd(g / (1.0 + exp(-g)) * linear(x, wu))
    return linear(h, wd)


def router(x: np.ndarray, wr: np.ndarray, k: int, norm_topk: bool):
    """Router of one layer for tokens x [T, H]: logits = Wr x (src/engine/tq_moe.c:612-618);
    p = softmax over all experts; the k largest (ties to the lowest index); weights p[sel],
    divided by their sum if norm_topk.  The reference picks the k largest logits and takes a
    softmax over them (:630-678), which is the norm_topk=true case of this formula; it breaks
    exact ties toward the highest index, this library toward the lowest.
    Returns (ids [T,k], weights [T,k], margin [T]): margin is the gap between the k-th and the
    (k+1)-th largest logit divided by the spread (standard deviation) of the token's logits: the
    distance of the choice from a flip, in the unit in which rounding moves the logits."""
    logits = linear(x, wr)
    p = softmax(logits)
    order = np.argsort(-p, axis=-1, kind="stable")
    ids = order[:, :k]
    w = np.take_along_axis(p, ids, axis=-1)
    if p.shape[1] > k:
        margin = (np.take_along_axis(logits, order[:, k - 1:k], axis=-1)
                  - np.take_along_axis(logits, order[:, k:k + 1], axis=-1))[:, 0] / (logits.std(axis=-1) + 1e-30)
    else:
        margin = np.full(p.shape[0], np.inf)
    if norm_topk:
        w = w / w.sum(axis=-1, keepdims=True)
    return ids, w, margin


def moe_feed_forward(m: PlainModel, l: int, x: np.ndarray, rnd: Round = no_round,
                     forced_ids: Optional[np.ndarray] = None, record: Optional[dict] = None) -> np.ndarray:
    """Routed experts in the order chosen, then the shared expert scaled by a sigmoid gate
    (src/engine/tq_moe.c:688-1059: route :704-716, experts :864-1000, shared :1006-1058)."""
    p = f"model.layers.{l}.mlp."
    w = m.w
    ids, wts, margin = router(x, w[p + "gate.weight"], m.k, m.norm_topk)
    if forced_ids is not None:
        probs = softmax(linear(x, w[p + "gate.weight"]))
        ids = forced_ids
        wts = np.take_along_axis(probs, ids, axis=-1)
        if m.norm_topk:
            wts = wts / wts.sum(axis=-1, keepdims=True)
    if record is not None:
        record.setdefault("ids", {})[l] = ids
        record.setdefault("weights", {})[l] = wts
        record.setdefault("margin", {})[l] = margin
    y = np.zeros_like(x)
    for e in np.unique(ids):                 # expert by expert: each one's weights are fetched once
        rows, cols = np.nonzero(ids == e)    # a token chooses an expert at most once
        pe = f"{p}experts.{int(e)}."
        o = swiglu(x[rows], w[pe + "gate_proj.weight"], w[pe + "up_proj.weight"],
                   w[pe + "down_proj.weight"], rnd, MOE_EXP)
        y[rows] += wts[rows, cols][:, None] * o
    if m.cfg.get("shared_expert_intermediate_size", 0) > 0:
        s = 1.0 / (1.0 + MOE_EXP(-linear(x, w[p + "shared_expert_gate.weight"])))      # [T,1]
        o = swiglu(x, w[p + "shared_expert.gate_proj.weight"], w[p + "shared_expert.up_proj.weight"],
                   w[p + "shared_expert.down_proj.weight"], rnd, MOE_EXP)
        y = y + s * o
    return y


def dense_feed_forward(m: PlainModel, l: int, x: np.ndarray, rnd: Round = no_round) -> np.ndarray:
    """A layer without a router is a dense SwiGLU (src/engine/tq_transformer.c:2707-2824)."""
    p = f"model.layers.{l}.mlp."
    return swiglu(x, m.w[p + "gate_proj.weight"], m.w[p + "up_proj.weight"], m.w[p + "down_proj.weight"], rnd)


def attention_mixer(m: PlainModel, l: int, x: np.ndarray, positions: np.ndarray, rnd: Round = no_round,
                    pairing: str = "half") -> np.ndarray:
    """QKV with bias, rotary on q and k, attention, output projection
    (src/engine/tq_transformer.c:1027-1093, 1343, 1909-2191, 2231-2240)."""
    p = f"model.layers.{l}.self_attn."
    w = m.w
    T = x.shape[0]
    q = rnd(linear(x, w[p + "q_proj.weight"])) + w.get(p + "q_proj.bias", 0.0)
    k = rnd(linear(x, w[p + "k_proj.weight"])) + w.get(p + "k_proj.bias", 0.0)
    v = rnd(linear(x, w[p + "v_proj.weight"])) + w.get(p + "v_proj.bias", 0.0)
    q = rnd(rotary(q.reshape(T, m.nh, m.hd), positions, m.theta, pairing))
    k = rnd(rotary(k.reshape(T, m.nkv, m.hd), positions, m.theta, pairing))
    v = rnd(v.reshape(T, m.nkv, m.hd))
    o = rnd(attention(q, k, v, m.layer_window(l)))
    return linear(o, w[p + "o_proj.weight"])


def block(m: PlainModel, l: int, x: np.ndarray, positions: np.ndarray, rnd: Round = no_round,
          pairing: str = "half", forced_ids=None, record=None) -> np.ndarray:
    """norm -> mixer -> add; norm -> feed-forward -> add
    (src/engine/tq_transformer.c:2494, 2268, 2685, 2701)."""
    p = f"model.layers.{l}."
    xn = rnd(rmsnorm(x, m.w[p + "input_layernorm.weight"], m.eps))
    x = x + attention_mixer(m, l, xn, positions, rnd, pairing)
    xn = rnd(rmsnorm(x, m.w[p + "post_attention_layernorm.weight"], m.eps))
    if m.layer_is_sparse(l):
        y = moe_feed_forward(m, l, xn, rnd, None if forced_ids is None else forced_ids[l], record)
    else:
        y = dense_feed_forward(m, l, xn, rnd)
    return x + y


def forward(m: PlainModel, tokens: Sequence[int], rnd: Round = no_round, pairing: str = "half",
            forced_ids=None, record=None, rows: Optional[Sequence[int]] = None) -> np.ndarray:
    """Logits [T, V] of one whole sequence (src/engine/tq_transformer.c:2281-3029:
    embedding, layers, final norm :2922, logits :2931-2942; a model without lm_head.weight
    reuses the embedding, src/engine/tq_model.c:1499-1516).  rows: the positions whose logits are wanted
    ([len(rows), V] comes back; the layers still run on every position)."""
    positions = np.arange(len(tokens))
    x = embedding(m.w["model.embed_tokens.weight"], tokens)
    for l in range(m.L):
        x = block(m, l, x, positions, rnd, pairing, forced_ids, record)
    if rows is not None:
        x = x[np.asarray(rows, dtype=np.int64)]
    xn = rnd(rmsnorm(x, m.w["model.norm.weight"], m.eps))
    head = m.w["model.embed_tokens.weight"] if m.tied else m.w["lm_head.weight"]
    return linear(xn, head)


# ------------------------------------------------------------------------------------
# sampling and generation
# ------------------------------------------------------------------------------------
def sample_argmax(logits: np.ndarray) -> int:
    """The first maximum wins (src/engine/tq_generate.c:30-40)."""
    return int(np.argmax(logits))


def uniform_for(seed: int, sequence: int, step: int) -> float:
    """The library's own counter-based stream: one uniform in [0,1) for (seed, sequence index,
    step), so that a draw does not depend on what else is in the batch.  (The reference keeps one
    xorshift64* state per generation call, src/engine/tq_generate.c:53-58.)  The mixing function
    is splitmix64 over seed, sequence and step; the top 24 bits make the float."""
    M = (1 << 64) - 1
    z = (int(seed) * 0x9E3779B97F4A7C15 + int(sequence) * 0xBF58476D1CE4E5B9 + int(step) * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & M
    for _ in range(2):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        z = z ^ (z >> 31)
    return float(z >> 40) / float(1 << 24)


def sample_top_p(logits: np.ndarray, temperature: float, top_p: float, u: float) -> int:
    """Temperature and nucleus sampling (src/engine/tq_generate.c:81-156): argmax if
    temperature <= 0 or top_p <= 0; keep logits >= max - 16*T; p = exp((l - max)/T) normalised;
    sort by p descending (ties: lower id first); cut where the cumulative sum reaches top_p;
    draw r = u * cumulative and walk the sorted list until the running sum reaches r."""
    if temperature <= 0.0 or top_p <= 0.0:
        return sample_argmax(logits)
    l = np.asarray(logits, dtype=np.float64)
    mx = l.max()
    keep = np.nonzero(l >= mx - 16.0 * temperature)[0]
    p = np.exp((l[keep] - mx) / temperature)
    p = p / p.sum()
    order = np.argsort(-p, kind="stable")
    ps, ids = p[order], keep[order]
    cum = np.cumsum(ps)
    n_top = int(np.searchsorted(cum, top_p, side="left")) + 1
    n_top = min(n_top, len(ps))
    r = u * cum[n_top - 1]
    j = int(np.searchsorted(cum[:n_top], r, side="left"))
    return int(ids[min(j, n_top - 1)])


def repetition_penalty(logits: np.ndarray, recent: Sequence[int], penalty: float) -> np.ndarray:
    """The reference lowers the logits of the tokens it saw last before it samples
    (src/engine/tq_generate.c:586-600; before the first sample :386-399): for each of them, once per
    occurrence, a positive logit is divided by the penalty and any other multiplied by it (float32)."""
    out = np.array(logits, dtype=np.float32, copy=True)
    p = np.float32(penalty)
    for tok in recent:
        if 0 <= tok < out.shape[0]:
            out[tok] = out[tok] / p if out[tok] > 0 else out[tok] * p
    return out


def recent_tokens(prompt: Sequence[int], generated: Sequence[int], window: int) -> List[int]:
    """What the penalty looks at: the last `window` (at most 128) tokens of the prompt followed by the
    generated ones (src/engine/tq_generate.c:365-367, 381-384, 607-609)."""
    window = min(int(window), 128)
    return (list(prompt) + list(generated))[-window:] if window > 0 else []


def closes_a_loop(prompt: Sequence[int], generated: Sequence[int], window: int = 32) -> bool:
    """Whether the last of `generated` closes a repetition loop as the reference sees it
    (src/engine/tq_generate.c:370-384, 610-630): from the second sampled token on, the last four tokens
    (the last `window` tokens of the prompt count) are hashed, h = h * 31 + token in 32 bits, and compared
    with the hashes of up to 64 draws before; three matches are a loop.  Recomputed from scratch here."""
    tail = list(prompt)[-min(int(window), 128):] if window > 0 else []
    hashes = []
    for n in range(2, len(generated) + 1):
        seen = (tail + list(generated[:n]))[-128:]
        if len(seen) < 4:
            continue
        h = 0
        for t in seen[-4:]:
            h = (h * 31 + t) % (1 << 32)
        hashes.append(h)
    if not hashes or len(generated) < 2 or len((tail + list(generated))[-128:]) < 4:
        return False
    return hashes[:-1][-64:].count(hashes[-1]) >= 3


def generate(m: PlainModel, prompt: Sequence[int], max_new_tokens: int, temperature: float = 0.0,
             top_p: float = 1.0, seed: int = 0, sequence: int = 0, stop: Sequence[int] = (),
             rnd: Round = no_round, rep_penalty: float = 1.0, rep_window: int = 32) -> List[int]:
    """Greedy or sampled continuation by recomputing the whole sequence for every token
    (loop of src/engine/tq_generate.c:441-605 without loop detector or text stops; the repetition
    penalty :586-600 when rep_penalty > 1).  A stop token ends the sequence and is part of the output."""
    toks = list(prompt)
    out: List[int] = []
    for step in range(max_new_tokens):
        logits = forward(m, toks, rnd)[-1]
        if rep_penalty > 1.0:
            logits = repetition_penalty(logits, recent_tokens(prompt, out, rep_window), rep_penalty)
        if temperature <= 0.0:
            t = sample_argmax(logits)
        else:
            t = sample_top_p(logits, temperature, top_p, uniform_for(seed, sequence, step))
        out.append(t)
        toks.append(t)
        if t in stop:
            break
    return out
