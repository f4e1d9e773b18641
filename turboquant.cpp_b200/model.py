"""The Python entry point: a model folder in, generated token ids out.

In the manner of the reference's binding (bindings/python/quantcpp/__init__.py:220-676):
``Model(path, temperature=…, top_p=…, max_tokens=…, context_length=…)`` with ``ask`` for one
answer, ``generate`` as an iterator of pieces, ``close`` and use as a context manager, and
``FileNotFoundError`` for a path that does not exist.  The reference's methods take and return
text through its tokenizer; this library's unit is the token id, so prompts are lists of ids and
answers are lists of ids.  ``generate_batch`` is this library's addition: several prompts of
unequal lengths as batches.
"""
from __future__ import annotations

import os
from typing import Iterator, List, Optional, Sequence, Union

import torch

from .engine.generate import GenParams, GenResult, GenStats, generate as _generate
from .engine.loading import load_model
from .cache import PAGE_SIZE
from .engine.step import Engine
from .sampling import Sampler


class Model:
    def __init__(self, path: str, *, temperature: float = 0.7, top_p: float = 0.9, max_tokens: int = 256,
                 context_length: int = 0, seed: int = 42, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_batch: int = 8, stop_token_ids: Optional[Sequence[int]] = None, rep_penalty: float = 1.0,
                 rep_window: int = 32, detect_loops: bool = False):
        """path: folder with config.json and safetensors.  context_length: most tokens one request
        may hold (0: the model's max_position_embeddings, capped at 4096 as the reference caps its
        default context, src/engine/tq_model.c:2951).  The cache is sized for max_batch such requests.
        rep_penalty > 1 lowers the logits of a request's last rep_window tokens before each draw, as the
        reference does with 1.1 over 32 tokens (include/turboquant/tq_engine.h:408-409); 1 (the default
        here) leaves the logits alone.  detect_loops ends a request when its last four tokens have come up three
        times among the 64 draws before, as the reference always does (src/engine/tq_generate.c:610-630)."""
        if not os.path.isdir(path):
            raise FileNotFoundError(f"model folder '{path}' does not exist")
        self._setup(load_model(path, dtype, device), path, temperature, top_p, max_tokens, context_length, seed,
                    device, max_batch, stop_token_ids, rep_penalty, rep_window, detect_loops)

    @classmethod
    def from_model(cls, model, *, temperature: float = 0.7, top_p: float = 0.9, max_tokens: int = 256,
                   context_length: int = 0, seed: int = 42, device: str = "cuda:0", max_batch: int = 8,
                   stop_token_ids: Optional[Sequence[int]] = None, rep_penalty: float = 1.0,
                   rep_window: int = 32, detect_loops: bool = False) -> "Model":
        """Wraps a model that is already on the device (for instance one with random weights)."""
        self = cls.__new__(cls)
        self._setup(model, "", temperature, top_p, max_tokens, context_length, seed, device, max_batch, stop_token_ids,
                    rep_penalty, rep_window, detect_loops)
        return self

    def _setup(self, model, path, temperature, top_p, max_tokens, context_length, seed, device, max_batch,
               stop_token_ids, rep_penalty=1.0, rep_window=32, detect_loops=False) -> None:
        self._path = path
        self.rep_penalty, self.rep_window, self.detect_loops = float(rep_penalty), int(rep_window), bool(detect_loops)
        self.temperature, self.top_p, self.max_tokens, self.seed = temperature, top_p, max_tokens, seed
        self.max_batch = int(max_batch)
        self._model = model
        ctx = int(context_length) if context_length and context_length > 0 else min(self._model.max_position, 4096)
        self.context_length = min(ctx, self._model.max_position)
        page = PAGE_SIZE
        per_request = -(-self.context_length // page) * page
        self._engine = Engine(self._model, max_tokens=per_request * self.max_batch, max_slots=max(self.max_batch, 1),
                              device=device)
        eos = getattr(self._model.config, "eos_token_ids", ())
        self.stop_token_ids = tuple(stop_token_ids) if stop_token_ids is not None else tuple(eos)
        self.last_stats: Optional[GenStats] = None
        self.last_results: List[GenResult] = []
        self._worker = self._worker_stop = None

    # ---- properties ---------------------------------------------------------------------------
    @property
    def path(self) -> str:
        return self._path

    @property
    def config(self):
        return self._model.config

    @property
    def engine(self) -> Engine:
        return self._engine

    def warm_up(self, batch_sizes: Optional[Sequence[int]] = None) -> List[int]:
        """Captures the decode steps of these batch sizes (default: 1..max_batch) before the first request, so that
        no request waits for a capture when its batch shrinks to a size not seen before.  Returns the sizes captured."""
        self._check_open()
        return self._engine.warm_up(range(1, self.max_batch + 1) if batch_sizes is None else batch_sizes)

    # ---- generation ---------------------------------------------------------------------------
    def _params(self, max_tokens, temperature, top_p, seed, stop_token_ids, rep_penalty=None, rep_window=None,
                detect_loops=None) -> GenParams:
        return GenParams(
            max_new_tokens=self.max_tokens if max_tokens is None else int(max_tokens),
            temperature=self.temperature if temperature is None else float(temperature),
            top_p=self.top_p if top_p is None else float(top_p),
            seed=self.seed if seed is None else int(seed),
            stop_token_ids=self.stop_token_ids if stop_token_ids is None else tuple(stop_token_ids),
            rep_penalty=self.rep_penalty if rep_penalty is None else float(rep_penalty),
            rep_window=self.rep_window if rep_window is None else int(rep_window),
            detect_loops=self.detect_loops if detect_loops is None else bool(detect_loops))

    def generate_batch(self, prompts: Sequence[Sequence[int]], *, max_tokens: Optional[int] = None,
                       temperature: Optional[float] = None, top_p: Optional[float] = None,
                       seed: Optional[int] = None, stop_token_ids: Optional[Sequence[int]] = None,
                       on_tokens=None, rep_penalty: Optional[float] = None,
                       rep_window: Optional[int] = None, detect_loops: Optional[bool] = None) -> List[List[int]]:
        """Continuations of several prompts (token ids in, token ids out, on the host)."""
        self._check_open()
        import threading
        if self._worker is not None and self._worker.is_alive() and threading.current_thread() is not self._worker:
            raise RuntimeError("a generate() of this model is still running; finish or close its iterator first")
        p = self._params(max_tokens, temperature, top_p, seed, stop_token_ids, rep_penalty, rep_window, detect_loops)
        stats = GenStats()
        sampler = Sampler(p.temperature, p.top_p, p.seed, p.rep_penalty, p.rep_window)
        results = _generate(self._engine, sampler, prompts, p, self.max_batch,
                            on_tokens=on_tokens, stats=stats, sync=torch.cuda.synchronize)
        self._engine.check_kernels()
        self.last_stats = stats
        self.last_results = results
        return [r.tokens for r in results]

    def ask(self, prompt: Sequence[int], **kw) -> List[int]:
        """The whole continuation of one prompt."""
        return self.generate_batch([prompt], **kw)[0]

    def generate(self, prompt: Sequence[int], **kw) -> Iterator[int]:
        """Yields the continuation's tokens one by one as they are sampled.  The decoding runs in a thread of its
        own; a consumer that stops early (break, an exception, close()) stops it too: the thread is told at its
        next token, gives its sequences back and is joined before this generator, or close(), returns."""
        self._check_open()
        if self._worker is not None and self._worker.is_alive():
            raise RuntimeError("a generate() of this model is still running; finish or close its iterator first")
        import queue
        import threading
        q: "queue.Queue" = queue.Queue()
        done = object()
        stop = threading.Event()

        class _Stopped(Exception):
            pass

        def told(idx, toks):
            if stop.is_set():
                raise _Stopped()                 # unwinds through the generation loop, which closes its sequences
            for t in toks:
                q.put(t)

        def run():
            try:
                self.generate_batch([prompt], on_tokens=told, **kw)
                q.put(done)
            except _Stopped:
                q.put(done)
            except BaseException as e:  # noqa: BLE001 - handed to the consumer
                q.put(e)

        t = threading.Thread(target=run, daemon=True)
        self._worker, self._worker_stop = t, stop
        t.start()
        try:
            while True:
                item = q.get()
                if item is done:
                    break
                if isinstance(item, BaseException):
                    raise item
                yield item
        finally:
            stop.set()
            t.join()
            self._worker = None

    # ---- lifetime -----------------------------------------------------------------------------
    def _check_open(self) -> None:
        if self._engine is None:
            raise RuntimeError("the model is closed")

    def close(self) -> None:
        worker = getattr(self, "_worker", None)
        if worker is not None and worker.is_alive():          # an iterator that was dropped half way
            self._worker_stop.set()
            worker.join()
        self._worker = None
        if self._engine is not None:
            self._engine.release()
        self._engine = None
        self._model = None
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    def __enter__(self) -> "Model":
        return self

    def __exit__(self, *exc) -> None:
        self.close()
