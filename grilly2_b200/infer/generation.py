"""A decode loop with Hugging Face's ``generate()`` arguments over the int8
Llama/Qwen2 decoder — the counterpart of python/grilly/infer/generation.py:103-206
for batch 1 (the decoder here is the batch-1 decode step of the int8 full-step
configuration).

The loop is built B200-first: ONE captured CUDA graph holds the whole step —
embedding of the token the sampler left on the device, the 24 layers, the head,
the sampler — and the sampler writes its token where the next step's embedding
reads it and appends it to a device history. The host only replays; it reads
back a token per step when there is an end-of-sequence id to stop at (as the
reference reads back only the sampled ids, generation.py:173), and nothing at
all until the end otherwise. The prompt but for its last token goes through
``LlamaDecoder.prefill`` (all rows at once, causal attention over the cache);
the last token is the first step's input.
"""
from __future__ import annotations

from dataclasses import dataclass, fields, replace

import numpy as np

from .. import _C
from .sampling import Generator, Sampler

__all__ = ["GenerationConfig", "generate"]


@dataclass
class GenerationConfig:
    """The ``transformers.GenerationConfig`` fields the loop uses, with their defaults (generation.py:66-86)."""
    max_length: int = 20
    max_new_tokens: int | None = None
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int | None = 50
    top_p: float | None = 1.0
    repetition_penalty: float = 1.0
    eos_token_id: int | list | None = None
    pad_token_id: int | None = None
    num_beams: int = 1
    use_cache: bool = True


_FIELDS = {f.name for f in fields(GenerationConfig)}


def generate(model, inputs=None, generation_config: GenerationConfig | None = None, *, generator: Generator | None = None,
             graphed: bool = True, **kwargs) -> np.ndarray:
    """``model``: a ``LlamaDecoder`` with an empty cache. ``inputs``: the prompt's token ids, int [1, length] (or a flat
    list). Returns the sequence, prompt first, as int64 [1, length]; a sequence that ended at ``eos_token_id`` stops
    there. Unknown keyword arguments raise, naming them, as the reference does."""
    if inputs is None:
        inputs = kwargs.pop("input_ids", None)
    if inputs is None:
        raise ValueError("generate() needs `inputs` (or `input_ids`): the prompt's token ids")
    ids = np.asarray(inputs)
    if ids.ndim == 1:
        ids = ids[None]
    if ids.ndim != 2 or ids.shape[0] != 1 or ids.shape[1] == 0 or not np.issubdtype(ids.dtype, np.integer):
        raise ValueError(f"`inputs` must be integer (1, length) with length > 0 (this decoder runs batch 1), got {ids.dtype} {ids.shape}")
    config = replace(generation_config or GenerationConfig())
    unused = [k for k in kwargs if k not in _FIELDS]
    if unused:
        raise ValueError(f"The following `model_kwargs` are not used by the model: {unused}")
    for k, v in kwargs.items():
        setattr(config, k, v)
    if config.num_beams != 1:
        raise NotImplementedError("grilly: generate() with num_beams > 1 (beam search) is not implemented yet")
    if not config.use_cache:
        raise NotImplementedError("grilly: generate(use_cache=False) is not implemented yet")
    prompt = ids.shape[1]
    total = prompt + config.max_new_tokens if config.max_new_tokens is not None else config.max_length
    steps = total - prompt
    if steps <= 0:
        return ids.astype(np.int64)
    cfg = model.cfg
    if total > cfg.max_cache_len + 1:
        raise RuntimeError(f"the cache holds {cfg.max_cache_len} positions; prompt + new tokens = {total}")
    eos = config.eos_token_id
    eos = set() if eos is None else {int(eos)} if isinstance(eos, (int, np.integer)) else {int(e) for e in eos}

    sampler = Sampler(1, cfg.vocab_size, do_sample=config.do_sample, temperature=config.temperature, top_k=config.top_k,
                      top_p=config.top_p, repetition_penalty=config.repetition_penalty, history_capacity=total,
                      draws=max(steps, 1), generator=generator)
    token = _C.Tensor.from_numpy(ids[0, :1].astype(np.int32), persistent=True)  # the step's input; the sampler's output

    def step():
        logits, _ = model.step(token, want_argmax=False)
        sampler.sample(logits, out=token)  # chooses, writes the next input, appends to the device history

    import grilly2_b200 as g
    run = g.graphed(step) if graphed else step
    if prompt > 1:  # the prompt but for its last token: one pass over all its rows
        model.prefill(_C.Tensor.from_numpy(ids[0, :-1].astype(np.int32)))
        token.copy_(_C.Tensor.from_numpy(ids[0, -1:].astype(np.int32)))
    sampler.set_history(ids)
    done = 0
    for _ in range(steps):
        run()
        done += 1
        if eos and int(token.numpy()[0]) in eos:  # the one value read back per step
            break
    out = sampler.history.numpy()[0, :prompt + done]
    return out[None].astype(np.int64)
