"""Next-token selection on the device — the counterpart of the reference's
``grilly.infer.sampling`` (python/grilly/infer/sampling.py over
crates/grilly-infer/src/sampling.rs and shaders/g2-sample.glsl): Hugging
Face's processors in ``generate()``'s order (repetition penalty; with
``do_sample`` temperature, top-k, top-p) and the draw, in one kernel, so the
logits never leave the GPU.

What differs from the reference, and why: token ids are int32 (this backend has
float32 and int32 tensors), and the random numbers a draw uses are read from a
DEVICE buffer at a DEVICE counter (``Sampler``), so a captured decode step that
ends in the sampler replays correctly — the reference passes each row's uniform
number from the host at every call.
"""
from __future__ import annotations

import ctypes

import numpy as np

from .. import _C, _lib
from .._lib import check

__all__ = ["Generator", "Sampler", "next_token", "probabilities"]


class Generator:
    """A seedable source of uniform numbers in [0, 1) (float32), standing in for the reference's global generator
    (``grilly.manual_seed``)."""

    def __init__(self, seed: int = 0) -> None:
        self._rng = np.random.default_rng(seed)

    def manual_seed(self, seed: int) -> "Generator":
        self._rng = np.random.default_rng(seed)
        return self

    def uniform(self, shape) -> np.ndarray:
        return self._rng.random(shape, dtype=np.float32)


_default_generator = Generator(0)


class Sampler:
    """The device state one stream of draws needs: a block of uniform numbers (``draws`` rows of ``rows`` values,
    reused cyclically), the draw counter, an optional token history with its length, and the kernel's scratch.
    ``sample(logits)`` chooses every row's next token; called inside a capture it records one launch that keeps
    counting when replayed."""

    def __init__(self, rows: int, vocab: int, *, do_sample: bool = False, temperature: float = 1.0, top_k: int | None = 50,
                 top_p: float | None = 1.0, repetition_penalty: float = 1.0, history_capacity: int = 0, draws: int = 1024,
                 generator: Generator | None = None) -> None:
        self.rows, self.vocab = int(rows), int(vocab)
        self.do_sample, self.temperature = bool(do_sample), float(temperature)
        self.top_k = int(top_k or 0)
        self.top_p = 1.0 if top_p is None else float(top_p)
        self.penalty = 1.0 if repetition_penalty is None else float(repetition_penalty)
        gen = generator or _default_generator
        self.n_draws = max(int(draws), 1)
        self.uniforms = _C.Tensor.from_numpy(gen.uniform((self.n_draws, self.rows)), persistent=True)
        self.draw_count = _C.Tensor.from_numpy(np.zeros(1, dtype=np.int32), persistent=True)
        self.scratch = _C.Tensor.empty((2, self.rows, self.vocab), "float32", persistent=True)
        self.capacity = int(history_capacity)
        self.history = self.hist_len = None
        if self.capacity:
            self.history = _C.Tensor.from_numpy(np.full((self.rows, self.capacity), -1, dtype=np.int32), persistent=True)
            self.hist_len = _C.Tensor.from_numpy(np.zeros(1, dtype=np.int32), persistent=True)

    def set_history(self, ids: np.ndarray) -> None:
        """Install the tokens so far: int [rows, length]."""
        ids = np.asarray(ids, dtype=np.int32).reshape(self.rows, -1)
        if ids.shape[1] > self.capacity:
            raise RuntimeError(f"the history holds {self.capacity} tokens per row, got {ids.shape[1]}")
        full = np.full((self.rows, self.capacity), -1, dtype=np.int32)
        full[:, :ids.shape[1]] = ids
        self.history = _C.Tensor.from_numpy(full, persistent=True)
        self.hist_len = _C.Tensor.from_numpy(np.array([ids.shape[1]], dtype=np.int32), persistent=True)

    def sample(self, logits: "_C.Tensor", out: "_C.Tensor | None" = None, probs: "_C.Tensor | None" = None,
               append: bool = True) -> "_C.Tensor":
        if logits.numel() != self.rows * self.vocab or logits.offset:
            raise RuntimeError(f"expected (batch, vocab) = ({self.rows}, {self.vocab}) at offset 0, got {list(logits.shape)}")
        tokens = out if out is not None else _C.Tensor.empty((self.rows,), "int32")
        h = self.history
        check(_lib.load().gq_sample(
            _C.context(), logits.storage.handle, self.rows, self.vocab, h.storage.handle if h is not None else 0, self.capacity,
            self.hist_len.storage.handle if h is not None else 0, 1 if (append and h is not None) else 0, 1 if self.do_sample else 0,
            self.temperature, self.top_k, self.top_p, self.penalty, self.uniforms.storage.handle, self.n_draws,
            self.draw_count.storage.handle, self.scratch.storage.handle, tokens.storage.handle,
            probs.storage.handle if probs is not None else 0))
        return tokens


def _one_shot(logits, history, generator, probs, **kw):
    rows, vocab = logits.shape
    cap = 0 if history is None else int(np.asarray(history).shape[1])
    s = Sampler(rows, vocab, history_capacity=cap, draws=1, generator=generator, **kw)
    if history is not None:
        s.set_history(np.asarray(history))
    return s.sample(logits, probs=probs, append=False)


def next_token(logits: "_C.Tensor", history=None, *, do_sample: bool = False, temperature: float = 1.0, top_k: int | None = 50,
               top_p: float | None = 1.0, repetition_penalty: float = 1.0, generator: Generator | None = None) -> "_C.Tensor":
    """Every row's next token (int32; -1 where nothing can be drawn). ``history``: int array [rows, length] of the
    tokens so far, for the repetition penalty. python/grilly/infer/sampling.py ``next_token``."""
    return _one_shot(logits, history, generator, None, do_sample=do_sample, temperature=temperature, top_k=top_k, top_p=top_p,
                     repetition_penalty=repetition_penalty)


def probabilities(logits: "_C.Tensor", history=None, *, temperature: float = 1.0, top_k: int | None = 0, top_p: float | None = 1.0,
                  repetition_penalty: float = 1.0) -> "_C.Tensor":
    """The distribution a sampled token is drawn from, after the processors: float32 [rows, vocab], zero where a token
    was filtered out. python/grilly/infer/sampling.py ``probabilities``."""
    probs = _C.Tensor.empty(tuple(logits.shape), "float32")
    _one_shot(logits, history, None, probs, do_sample=True, temperature=temperature, top_k=top_k, top_p=top_p,
              repetition_penalty=repetition_penalty)
    return probs
