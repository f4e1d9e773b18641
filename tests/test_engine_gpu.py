"""The engine against the plain implementation on the GPU, in float32 and in bfloat16: each
request alone and whole; with the last 32 tokens one by one; in batches of unequal lengths whose
shorter requests end earlier, one batch after another so that slots and pages are used again;
long decoding; the first tokens of a sequence."""
import numpy as np
import pytest

from conftest import TINY
from replay_util import batched, check_against_plain, run_schedule, whole, with_tail

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
NAMES = ["A", "B", "C"]


@pytest.fixture(scope="module")
def engines(tiny_folders):
    import turboquant_cpp_b200 as tq
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            model = tq.load_model(tiny_folders[name], dtype, "cuda:0")
            cache[(name, dtype)] = tq.Engine(model, max_tokens=1024, record_routing=True)
        return cache[(name, dtype)]
    return get


def tokens_for(name, n, seed):
    V = TINY[name][0]["vocab_size"]
    return np.random.default_rng(seed).integers(0, V, size=n).tolist()


def max_len(name):
    return TINY[name][0]["max_position_embeddings"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request(engines, plain_models, name, dtype):
    eng = engines(name, dtype)
    toks = tokens_for(name, min(100, max_len(name)), 10)
    logits, routing = run_schedule(eng, *whole("r", toks))
    assert sorted(logits["r"]) == list(range(len(toks)))
    check_against_plain(plain_models[name], toks, logits["r"], routing.get("r", {}), dtype, f"{name} whole")
    eng.cache.book.check_invariants()
    assert eng.cache.book.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(engines, plain_models, name, dtype):
    eng = engines(name, dtype)
    toks = tokens_for(name, min(100, max_len(name)), 11)
    logits, routing = run_schedule(eng, *with_tail("r", toks, 32))
    check_against_plain(plain_models[name], toks, logits["r"], routing.get("r", {}), dtype, f"{name} tail")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(engines, plain_models, name, dtype):
    """Batch 1: prompts 5/11/17 with 8, 3 and 8 further tokens; batch 2 on the same engine right
    after it (its sequences get the slots and pages batch 1 gave back): prompts 1/9/40/70 with
    16, 2, 16 and 5 further tokens (70 is longer than Tiny B's window and than one page)."""
    eng = engines(name, dtype)
    free_before = [p.n_free for p in eng.cache.book.pools]
    plans = [({"a": (5, 8), "b": (11, 3), "c": (17, 8)}, 20),
             ({"d": (1, 16), "e": (9, 2), "f": (40, 16), "g": (70, 5)}, 30)]
    for batch, seed in plans:
        reqs = {r: tokens_for(name, p + d, seed + i) for i, (r, (p, d)) in enumerate(batch.items())}
        logits, routing = run_schedule(eng, *batched(reqs, {r: batch[r][0] for r in batch}))
        for r, toks in reqs.items():
            assert sorted(logits[r]) == list(range(len(toks)))
            check_against_plain(plain_models[name], toks, logits[r], routing.get(r, {}), dtype, f"{name} batch {r}")
        eng.cache.book.check_invariants()
        assert [p.n_free for p in eng.cache.book.pools] == free_before      # everything was given back


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(engines, plain_models, name, dtype):
    """A short prompt, then token by token up to the model's last position (several pages, and far
    beyond the window of the windowed layers)."""
    eng = engines(name, dtype)
    n = max_len(name)
    toks = tokens_for(name, n, 12)
    logits, routing = run_schedule(eng, *with_tail("r", toks, n - 3))
    assert len(logits["r"]) == n
    check_against_plain(plain_models[name], toks, logits["r"], routing.get("r", {}), dtype, f"{name} long")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(engines, plain_models, name, dtype):
    """Positions 0, 1, 2: a prompt of one token, then single tokens."""
    eng = engines(name, dtype)
    toks = tokens_for(name, 4, 13)
    logits, routing = run_schedule(eng, *with_tail("r", toks, 3))
    check_against_plain(plain_models[name], toks, logits["r"], routing.get("r", {}), dtype, f"{name} first")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_decode_steps_run_as_graphs_and_give_the_bits_of_eager_steps(engines, tiny_folders, name, dtype):
    """The strict comparisons above go through the path generation uses: decode steps of the shared engines are
    replays of captured CUDA graphs (with the experts' choices read from memory of the graph).  The same steps
    launched one kernel at a time give the same logits bit for bit."""
    import turboquant_cpp_b200 as tq
    eng = engines(name, dtype)
    toks = tokens_for(name, min(90, max_len(name)), 14)
    before = eng.graphs.replays
    graph_logits, graph_routing = run_schedule(eng, *with_tail("r", toks, 40))
    assert eng.graphs.replays - before >= 39                   # all but the first step of a new batch size
    eager = tq.Engine(eng.model, max_tokens=1024, use_graphs=False)
    assert eager.graphs is None
    eager_logits, eager_routing = run_schedule(eager, *with_tail("r", toks, 40))
    for p in range(len(toks)):
        assert np.array_equal(graph_logits["r"][p], eager_logits["r"][p]), f"position {p}"
    for li in graph_routing.get("r", {}):
        for p in range(len(toks)):
            assert np.array_equal(graph_routing["r"][li][p], eager_routing["r"][li][p])


def test_step_refuses_bad_input(engines):
    import turboquant_cpp_b200 as tq
    eng = engines("A", "float32")
    seq = eng.open()
    with pytest.raises(tq.StepError):
        eng.step([tq.StepEntry(seq, [256], [0])])                 # token outside the vocabulary
    with pytest.raises(tq.StepError):
        eng.step([tq.StepEntry(seq, [1, 2], [2])])                # wanted place outside the tokens
    with pytest.raises(tq.StepError):
        eng.step([tq.StepEntry(seq, list(range(129)), [])])       # beyond max_position_embeddings
    assert seq.length == 0
    eng.close(seq)
    eng.cache.book.check_invariants()


def test_warm_up_captures_the_decode_graphs_ahead_of_the_first_batch(tiny_folders):
    """After warm_up the first decode step of a batch size is already a replay, slots and pages are all back, and
    the logits are those of an engine that was not warmed up, bit for bit."""
    import turboquant_cpp_b200 as tq
    model = tq.load_model(tiny_folders["A"], "bfloat16", "cuda:0")
    warm = tq.Engine(model, max_tokens=1024, max_slots=4)
    free = [p.n_free for p in warm.cache.book.pools]
    assert warm.warm_up([1, 3]) == [1, 3]
    assert warm.warm_up([3, 2]) == [2]                        # 3 has its graph already
    assert [p.n_free for p in warm.cache.book.pools] == free
    warm.cache.book.check_invariants()
    assert warm.warm_up([9]) == []                            # more sequences than slots: nothing captured, nothing held
    assert [p.n_free for p in warm.cache.book.pools] == free
    cold = tq.Engine(model, max_tokens=1024, max_slots=4)
    toks = tokens_for("A", 40, 5)
    out = {}
    for name, eng in (("warm", warm), ("cold", cold)):
        before = eng.graphs.replays
        seqs = [eng.open() for _ in range(3)]
        eng.step([tq.StepEntry(s, toks[:20 + i], []) for i, s in enumerate(seqs)])
        rows = [eng.step([tq.StepEntry(s, [toks[30 + j]], [0]) for s in seqs]).float().cpu().numpy() for j in range(3)]
        out[name] = (rows, eng.graphs.replays - before)
        for s in seqs:
            eng.close(s)
    assert out["warm"][1] == 3 and out["cold"][1] == 2         # the cold engine's first step of this size ran eagerly
    for a, b in zip(out["warm"][0], out["cold"][0]):
        assert np.array_equal(a, b)
    warm.release()
    cold.release()
