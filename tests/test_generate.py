"""The generation loop's decisions with a stand-in engine (CPU): batching, stop tokens, sequences
that end earlier, one batch after another, slots given back."""
import numpy as np
import pytest

from turboquant_cpp_b200.cache import CacheBook, CacheFull
from turboquant_cpp_b200.engine.generate import GenParams, GenStats, generate, plan_batches
from turboquant_cpp_b200.sampling import uniforms_for
from plain.qwen2_moe_plain import uniform_for


class FakeEngine:
    """Next token = (sum of the sequence's tokens) % vocab; the bookkeeping is the real CacheBook."""
    page_size, max_position = 64, 300

    def __init__(self, capacity_tokens=64 * 64, max_slots=8, vocab=50):
        self.book = CacheBook([capacity_tokens // 64], [0], 64, max_slots)
        self.capacity_tokens, self.max_slots, self.vocab = capacity_tokens, max_slots, vocab
        self.sums, self.step_sizes, self.max_live = {}, [], 0

    def open(self):
        s = self.book.open()
        self.sums[s.id] = 0
        self.max_live = max(self.max_live, len(self.book.live))
        return s

    def close(self, seq):
        self.book.close(seq)

    @staticmethod
    def make_entry(seq, tokens, want=()):
        return (seq, list(tokens), list(want))

    def step(self, entries):
        self.book.reserve_all([e[0] for e in entries], [len(e[1]) for e in entries])
        rows = []
        for seq, toks, want in entries:
            self.sums[seq.id] += sum(toks)
            self.book.commit(seq, len(toks))
            assert want in ([len(toks) - 1], [0])
            row = np.zeros(self.vocab)
            row[self.sums[seq.id] % self.vocab] = 1.0
            rows.append(row)
        self.step_sizes.append(len(entries))
        self.book.check_invariants()
        return np.stack(rows)


class FakeAheadEngine(FakeEngine):
    """The stand-in with the optional run-ahead interface: a step launched from the samples, then kept or dropped."""
    can_step_ahead = True

    def __init__(self, *a, **k):
        super().__init__(*a, **k)
        self.pending, self.kept, self.dropped = None, 0, 0

    class Reader:
        def __init__(self, n):
            self.n = n

        def start(self, tokens):
            snap = [int(t) for t in tokens]
            assert len(snap) <= self.n
            return lambda: snap

    def token_reader(self, n):
        return self.Reader(n)

    def step(self, entries):
        assert self.pending is None, "a step while another, launched ahead, has neither been kept nor dropped"
        return super().step(entries)

    def step_ahead(self, seqs, tokens):
        assert self.pending is None
        self.book.reserve_all(list(seqs), [1] * len(seqs))
        self.pending = (list(seqs), [int(t) for t in tokens])
        rows = np.zeros((len(seqs), self.vocab))
        for r, (s, t) in enumerate(zip(*self.pending)):
            rows[r, (self.sums[s.id] + t) % self.vocab] = 1.0
        return rows

    def commit_ahead(self):
        seqs, toks = self.pending
        self.pending = None
        for s, t in zip(seqs, toks):
            assert s.id in self.book.live
            self.sums[s.id] += t
            self.book.commit(s, 1)
        self.step_sizes.append(len(seqs))
        self.kept += 1
        self.book.check_invariants()

    def drop_ahead(self):
        assert self.pending is not None
        self.pending = None
        self.dropped += 1

class ArgmaxSampler:
    def __init__(self):
        self.calls = []

    def sample(self, logits, requests, steps):
        self.calls.append((list(requests), list(steps)))
        return np.argmax(logits, axis=1)


def expected(prompt, n, vocab=50, stop=()):
    out, s = [], sum(prompt)
    for _ in range(n):
        t = s % vocab
        out.append(t)
        s += t
        if t in stop:
            break
    return out


def test_batches_of_unequal_prompts_and_early_ends():
    eng, smp = FakeEngine(), ArgmaxSampler()
    prompts = [[1, 2, 3], [4] * 11, [5] * 17, [7], [9, 9]]
    stats = GenStats()
    res = generate(eng, smp, prompts, GenParams(max_new_tokens=6, stop_token_ids=(24,)), max_batch=3, stats=stats)
    for p, r in zip(prompts, res):
        assert r.tokens == expected(p, 6, stop=(24,))
        assert r.finish_reason == ("stop" if r.tokens[-1] == 24 else "length")
    assert any(r.finish_reason == "stop" and len(r.tokens) < 6 for r in res)      # one ended earlier
    assert stats.batches == 2 and eng.max_live == 3
    assert eng.step_sizes[0] == 3 and min(eng.step_sizes) < 3                     # the batch shrank
    assert not eng.book.live and eng.book.pools[0].n_free == eng.book.pools[0].n  # everything was given back
    # the sampler saw each request under its own index and its own token count
    for reqs, steps in smp.calls:
        for i, s in zip(reqs, steps):
            assert 0 <= s < 6 and 0 <= i < len(prompts)
    assert stats.generated_tokens == sum(len(r.tokens) for r in res)
    assert stats.prompt_tokens == sum(len(p) for p in prompts)


@pytest.mark.parametrize("stop,max_new", [((), 6), ((24,), 6), ((24, 3, 7), 12), ((), 1), ((), 2)])
def test_running_one_step_ahead_changes_no_result(stop, max_new):
    prompts = [[1, 2, 3], [4] * 11, [5] * 17, [7], [9, 9], [3] * 290]
    plain_eng, ahead_eng = FakeEngine(), FakeAheadEngine()
    params = GenParams(max_new_tokens=max_new, stop_token_ids=stop)
    want = generate(plain_eng, ArgmaxSampler(), prompts, params, max_batch=3)
    seen = {}
    got = generate(ahead_eng, ArgmaxSampler(), prompts, params, max_batch=3,
                   on_tokens=lambda idx, toks: [seen.setdefault(i, []).append(t) for i, t in zip(idx, toks)])
    assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in want]
    assert [seen[i] for i in range(len(prompts))] == [r.tokens for r in got]
    assert ahead_eng.step_sizes == plain_eng.step_sizes                 # the same steps were committed
    assert ahead_eng.pending is None and not ahead_eng.book.live
    assert ahead_eng.book.pools[0].n_free == ahead_eng.book.pools[0].n
    if max_new > 2:
        assert ahead_eng.kept > 0
    if stop and any(r.finish_reason == "stop" and len(r.tokens) < max_new for r in want):
        assert ahead_eng.dropped > 0                                    # an early end voided a step launched ahead
    if not stop:
        assert ahead_eng.dropped == 0                                   # ends by length are foreseen: nothing is wasted


def test_a_full_cache_ends_run_ahead_like_a_plain_step():
    for cls in (FakeEngine, FakeAheadEngine):
        small = cls(capacity_tokens=128, max_slots=4)
        res = generate(small, ArgmaxSampler(), [[1] * 60, [2] * 60], GenParams(max_new_tokens=200), max_batch=4)
        assert [r.finish_reason for r in res] == ["context", "context"]
        assert all(len(r.tokens) == 128 - 60 + 1 for r in res)
        assert not small.book.live and getattr(small, "pending", None) is None


def test_an_error_in_the_callback_leaves_no_step_pending():
    eng = FakeAheadEngine()

    def boom(idx, toks):
        if len(toks) and eng.kept >= 1:
            raise RuntimeError("stop here")
    with pytest.raises(RuntimeError):
        generate(eng, ArgmaxSampler(), [[1, 2], [3]], GenParams(max_new_tokens=8), on_tokens=boom)
    assert eng.pending is None and not eng.book.live


def test_streaming_callback_gets_every_token_once():
    eng = FakeEngine()
    seen = {}
    prompts = [[1], [2, 2], [3, 3, 3]]
    res = generate(eng, ArgmaxSampler(), prompts, GenParams(max_new_tokens=4), max_batch=8,
                   on_tokens=lambda idx, toks: [seen.setdefault(i, []).append(t) for i, t in zip(idx, toks)])
    assert [seen[i] for i in range(3)] == [r.tokens for r in res]


def test_context_and_cache_limits_end_a_sequence():
    eng = FakeEngine()
    res = generate(eng, ArgmaxSampler(), [[1] * 298], GenParams(max_new_tokens=10))
    assert res[0].finish_reason == "context" and len(res[0].tokens) == 3         # 298 + 2 fed back = 300 positions
    small = FakeEngine(capacity_tokens=128, max_slots=4)
    res = generate(small, ArgmaxSampler(), [[1] * 60, [2] * 60], GenParams(max_new_tokens=200), max_batch=4)
    assert [r.finish_reason for r in res] == ["context", "context"]             # each alone, until the cache is full
    assert all(len(r.tokens) == 128 - 60 + 1 for r in res)
    assert not small.book.live
    with pytest.raises(CacheFull):
        generate(small, ArgmaxSampler(), [[1] * 200], GenParams(max_new_tokens=1))
    with pytest.raises(ValueError):
        generate(eng, ArgmaxSampler(), [[]], GenParams(max_new_tokens=1))
    assert generate(eng, ArgmaxSampler(), [[1]], GenParams(max_new_tokens=0))[0].tokens == []


def test_plan_batches_respects_slots_pages_and_order():
    plan = plan_batches([10, 100, 20, 64, 5], max_new_tokens=30, max_batch=8, capacity_tokens=256, max_slots=8,
                        page_size=64, max_position=1000)
    assert plan == [[0], [1, 2], [3], [4]] or sum(plan, []) == [0, 1, 2, 3, 4]
    assert sum(plan, []) == [0, 1, 2, 3, 4]
    for b in plan:
        assert sum(-(-(n + 30) // 64) for n in ([10, 100, 20, 64, 5][i] for i in b)) <= 4
    assert plan_batches([1] * 5, 1, max_batch=2, capacity_tokens=6400, max_slots=8, page_size=64, max_position=100) == \
        [[0, 1], [2, 3], [4]]
    assert plan_batches([1] * 5, 1, max_batch=8, capacity_tokens=6400, max_slots=3, page_size=64, max_position=100) == \
        [[0, 1, 2], [3, 4]]


def test_uniforms_do_not_depend_on_the_batch_and_match_the_plain_stream():
    a = uniforms_for(7, [0, 1, 2, 3], [5, 5, 5, 5])
    b = uniforms_for(7, [2], [5])
    assert a[2] == b[0] and len(set(a.tolist())) == 4
    assert all(0.0 <= u < 1.0 for u in a)
    for seed, r, s in [(7, 2, 5), (0, 0, 0), (42, 63, 4095), (2 ** 40 + 3, 9, 1)]:
        assert float(uniforms_for(seed, [r], [s])[0]) == pytest.approx(uniform_for(seed, r, s), abs=0)
    many = uniforms_for(1, np.arange(20000) % 64, np.arange(20000) // 64)
    assert abs(many.mean() - 0.5) < 0.01 and abs(np.mean(many < 0.1) - 0.1) < 0.01


class PenalizingSampler(ArgmaxSampler):
    """A sampler that asks for each request's tokens so far, as the library's does with a repetition penalty."""
    penalizes = True

    def __init__(self):
        super().__init__()
        self.seen = []

    def sample(self, logits, requests, steps, recent=None):
        assert recent is not None and len(recent) == len(requests)
        self.seen.append({i: list(r) for i, r in zip(requests, recent)})
        return super().sample(logits, requests, steps)


@pytest.mark.parametrize("engine", [FakeEngine, FakeAheadEngine])
def test_a_penalizing_sampler_is_handed_each_requests_tokens_so_far(engine):
    """Prompt first, then everything generated before this draw, per request, whether or not the engine runs a
    step ahead and whichever requests are left in the batch; a sampler that does not ask gets no such argument."""
    prompts = [[1, 2, 3], [4] * 11, [7]]
    smp = PenalizingSampler()
    res = generate(engine(), smp, prompts, GenParams(max_new_tokens=5, stop_token_ids=(24,)), max_batch=3)
    plain = generate(engine(), ArgmaxSampler(), prompts, GenParams(max_new_tokens=5, stop_token_ids=(24,)), max_batch=3)
    assert [r.tokens for r in res] == [r.tokens for r in plain]
    draws = {i: 0 for i in range(len(prompts))}
    for call in smp.seen:
        for i, recent in call.items():
            assert recent == prompts[i] + res[i].tokens[:draws[i]]
            draws[i] += 1
    assert all(draws[i] == len(res[i].tokens) for i in draws)


def test_sampler_settings_for_the_penalty():
    from turboquant_cpp_b200.sampling import Sampler
    assert not Sampler(0.0).penalizes and not Sampler(0.7, 0.9, 1, rep_penalty=1.0).penalizes
    s = Sampler(0.0, rep_penalty=1.1, rep_window=1000)
    assert s.penalizes and s.rep_window == 128            # the reference keeps at most 128 recent tokens
    assert not Sampler(0.0, rep_penalty=1.1, rep_window=0).penalizes
    assert GenParams().rep_penalty == 1.0 and GenParams().rep_window == 32


def test_random_requests_give_the_same_results_with_and_without_running_ahead():
    """Many random mixes of prompt lengths, stop tokens, limits, batch sizes and cache sizes: the loop over the
    plain stand-in and over the one that runs a step ahead give every request the tokens of its own closed-form
    continuation (cut by a stop token, the limit, the model's positions or a full cache), commit the same steps,
    and leave nothing held."""
    import random
    rng = random.Random(5)
    for case in range(150):
        n = rng.randint(1, 9)
        prompts = [[rng.randrange(50) for _ in range(rng.choice([1, 2, 3, 17, 63, 64, 65, 120]))] for _ in range(n)]
        stop = tuple(rng.sample(range(50), rng.choice([0, 0, 1, 3, 10])))
        params = GenParams(max_new_tokens=rng.choice([1, 2, 3, 8, 40]), stop_token_ids=stop)
        max_batch = rng.choice([1, 2, 3, 8])
        pages = rng.choice([4, 6, 16, 64])
        slots = rng.choice([1, 2, 8])
        engines = [FakeEngine(capacity_tokens=64 * pages, max_slots=slots), FakeAheadEngine(capacity_tokens=64 * pages, max_slots=slots)]
        runs = [generate(e, ArgmaxSampler(), prompts, params, max_batch=max_batch) for e in engines]
        a, b = ([(r.tokens, r.finish_reason) for r in run] for run in runs)
        assert a == b, f"case {case}"
        assert engines[0].step_sizes == engines[1].step_sizes, f"case {case}"
        for e in engines:
            assert not e.book.live and e.book.pools[0].n_free == e.book.pools[0].n and e.book.slots.n_held == 0
            assert e.max_live <= min(max_batch, slots)
        assert engines[1].pending is None
        for p, (toks, why) in zip(prompts, a):
            full = expected(p, params.max_new_tokens, stop=stop)
            assert toks == full[:len(toks)] and len(toks) >= 1, f"case {case}"
            if why == "stop":
                assert toks[-1] in stop and toks == full
            elif why == "length":
                assert len(toks) == params.max_new_tokens
            else:
                assert why == "context" and len(toks) < params.max_new_tokens       # positions or pages ran out


def test_loop_detector_ends_a_request_as_the_reference_does():
    """Off by default.  On, a request ends with 'loop' at the first token whose 4-gram has come up three times among
    the 64 draws before, and that token is not part of the output; the plain restatement, which recomputes
    everything from the tokens, names the same place; other requests of the batch go on."""
    from plain.qwen2_moe_plain import closes_a_loop
    from turboquant_cpp_b200.engine.generate import LoopDetector
    prompts = [[0], [1, 2, 3], [25, 25]]           # 0 -> 0 0 0 ... ; 25+25 = 50 -> 0 0 0 ...
    for cls in (FakeEngine, FakeAheadEngine):
        off = generate(cls(), ArgmaxSampler(), prompts, GenParams(max_new_tokens=30), max_batch=4)
        assert all(r.finish_reason == "length" and len(r.tokens) == 30 for r in off)
        seen = {}
        on = generate(cls(), ArgmaxSampler(), prompts, GenParams(max_new_tokens=30, detect_loops=True), max_batch=4,
                      on_tokens=lambda idx, toks: [seen.setdefault(i, []).append(t) for i, t in zip(idx, toks)])
        for p, r, full in zip(prompts, on, off):
            assert r.tokens == full.tokens[:len(r.tokens)] and seen[prompts.index(p)] == r.tokens
            if r.finish_reason == "loop":
                n = len(r.tokens)
                assert closes_a_loop(p, full.tokens[:n + 1]) and not any(closes_a_loop(p, full.tokens[:k]) for k in range(1, n + 1))
            else:
                assert r.finish_reason == "length" and not any(closes_a_loop(p, full.tokens[:k]) for k in range(1, 31))
        assert on[0].finish_reason == "loop" and on[2].finish_reason == "loop"
    # the detector against the restatement on random tokens from a small alphabet (loops are frequent)
    import random
    rng = random.Random(3)
    for _ in range(200):
        prompt = [rng.randrange(3) for _ in range(rng.choice([0, 1, 2, 5, 40, 200]))]
        det, out = LoopDetector(prompt, 32), []
        for _ in range(120):
            out.append(rng.randrange(3))
            assert det.push(out[-1]) == closes_a_loop(prompt, out)
