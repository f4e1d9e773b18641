"""The Python entry point's and the command line's plumbing, with stand-ins for the device side (CPU): every
option reaches the generation loop and the sampler under its own name, and the results come back."""
import types

import numpy as np
import pytest

import turboquant_cpp_b200.model as model_module
from test_generate import ArgmaxSampler, FakeAheadEngine, expected


class StandInEngine(FakeAheadEngine):
    made = []

    def __init__(self, model, max_tokens, max_slots=None, device="cuda:0"):
        super().__init__(capacity_tokens=max_tokens, max_slots=max_slots or 8)
        self.max_position = model.max_position
        self.released = False
        StandInEngine.made.append(self)

    def check_kernels(self):
        pass

    def release(self):
        self.released = True


class StandInSampler(ArgmaxSampler):
    made = []

    def __init__(self, temperature, top_p, seed, rep_penalty=1.0, rep_window=32):
        super().__init__()
        self.args = (temperature, top_p, seed, rep_penalty, rep_window)
        self.penalizes = rep_penalty > 1.0
        self.recents = []
        StandInSampler.made.append(self)

    def sample(self, logits, requests, steps, recent=None):
        assert (recent is not None) == self.penalizes
        self.recents.append(recent)
        return super().sample(logits, requests, steps)


@pytest.fixture
def stand_ins(monkeypatch, tmp_path):
    StandInEngine.made.clear()
    StandInSampler.made.clear()
    fake_model = types.SimpleNamespace(max_position=300, config=types.SimpleNamespace(eos_token_ids=(24,)))
    monkeypatch.setattr(model_module, "load_model", lambda path, dtype, device: fake_model)
    monkeypatch.setattr(model_module, "Engine", StandInEngine)
    monkeypatch.setattr(model_module, "Sampler", StandInSampler)
    monkeypatch.setattr(model_module.torch.cuda, "synchronize", lambda *a, **k: None)
    return str(tmp_path)


def test_model_options_reach_the_loop_and_the_sampler(stand_ins):
    prompts = [[1, 2, 3], [0], [9, 9]]
    with model_module.Model(stand_ins, temperature=0.3, top_p=0.8, max_tokens=12, seed=5, max_batch=2,
                            context_length=100, rep_penalty=1.2, rep_window=7, detect_loops=True) as m:
        eng = StandInEngine.made[-1]
        assert m.context_length == 100 and eng.capacity_tokens == 128 * 2 and eng.max_slots == 2
        assert m.stop_token_ids == (24,)                                   # the configuration's end-of-sequence ids
        outs = m.generate_batch(prompts)
        smp = StandInSampler.made[-1]
        assert smp.args == (0.3, 0.8, 5, 1.2, 7) and all(r is not None for r in smp.recents)
        assert m.last_stats.batches == 2                                   # two requests at a time
        for p, o, r in zip(prompts, outs, m.last_results):
            full = expected(p, 12, stop=(24,))
            assert o == full[:len(o)] and r.tokens == o
        assert m.last_results[1].finish_reason == "loop"                   # 0 0 0 0 ...
        # per-call overrides
        plain = m.generate_batch(prompts, rep_penalty=1.0, detect_loops=False, max_tokens=5, stop_token_ids=[])
        assert StandInSampler.made[-1].args[3] == 1.0 and all(r is None for r in StandInSampler.made[-1].recents)
        assert plain == [expected(p, 5) for p in prompts]
        assert m.ask([4, 4], max_tokens=3, detect_loops=False) == expected([4, 4], 3)
        assert list(m.generate([4, 4], max_tokens=3, detect_loops=False)) == expected([4, 4], 3)
        assert not eng.book.live
    assert eng.released
    with pytest.raises(RuntimeError):
        m.ask([1])
    with pytest.raises(FileNotFoundError):
        model_module.Model(stand_ins + "/nowhere")


def test_command_line_options_reach_the_model(stand_ins, monkeypatch, capsys):
    import turboquant_cpp_b200.cli as cli
    monkeypatch.setattr(cli, "parse_ids", cli.parse_ids)
    import torch
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    rc = cli.main([stand_ins, "-p", "1,2,3", "-p", "0", "-n", "6", "-T", "0", "-s", "0", "--rep-penalty", "1.1",
                   "--rep-window", "9", "--detect-loops", "--stop", "24", "--batch", "4", "--ctx", "64"])
    assert rc == 0
    out, err = capsys.readouterr()
    lines = [[int(t) for t in l.split()] for l in out.strip().splitlines()]
    assert lines[0] == expected([1, 2, 3], 6, stop=(24,)) and lines[1] == expected([0], 6)[:len(lines[1])]
    assert "tokens in" in err and "tok/s" in err
    assert StandInSampler.made[-1].args == (0.0, 0.9, 42, 1.1, 9)          # seed 0 means the default, 42
    assert StandInEngine.made[-1].capacity_tokens == 64 * 4
    assert cli.parse_ids("1, 2 3") == [1, 2, 3]
    with pytest.raises(SystemExit):
        cli.parse_ids("1,x")


def test_a_dropped_iterator_stops_its_decoding_and_gives_everything_back(stand_ins):
    m = model_module.Model(stand_ins, temperature=0.0, max_tokens=200, max_batch=2, context_length=250,
                           stop_token_ids=[])
    eng = StandInEngine.made[-1]
    import time
    slow = eng.step_ahead
    eng.step_ahead = lambda *a: (time.sleep(0.002), slow(*a))[1]        # 200 tokens take 0.4 s and more
    it = m.generate([5, 6, 7], detect_loops=False)
    first = [next(it), next(it), next(it)]
    assert first == expected([5, 6, 7], 3)
    with pytest.raises(RuntimeError, match="still running"):
        m.ask([1])                                    # one generation at a time on one engine
    it.close()                                        # the consumer walks away
    assert m._worker is None and not eng.book.live    # the thread has ended and its sequence is closed
    assert len(eng.step_sizes) < 100                  # long before the 200 tokens it was asked for
    assert m.ask([4, 4], max_tokens=3) == expected([4, 4], 3)      # the model is usable again
    it = m.generate([5, 6, 7], detect_loops=False)
    next(it)
    m.close()                                         # close() with an iterator half way: stops and joins it
    assert eng.released and not eng.book.live
