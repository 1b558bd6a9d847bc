"""The Python entry point.

    from gguf2bin_b200.api import LLM
    llm = LLM("model_dir", dtype="bfloat16", max_tokens=65536)
    outs = llm.generate([[1, 2, 3], [4, 5]], n=64, temperature=0.0)

Options carry the names and defaults of the reference's ``run`` command
(src/main.c:65-94, 273 of AnonymoDGH/gguf2bin): ``n`` new tokens (64), ``temperature``
(0.7; 0 is greedy), ``top_k`` (40), ``top_p`` (0.9), ``repeat_penalty`` (1.1), ``ctx``
(context limit; the model's by default).  Token ids go in and come out; there is no
tokenizer.  ``seed`` makes sampling reproducible (the reference seeds from the clock,
src/main.c:315).
"""
from __future__ import annotations

from typing import Optional, Sequence

from .engine.backend import EngineBackend
from .engine.generate import Generation, generate
from .engine.model import Model
from .engine.step import Engine, StepEntry
from .sampling import SamplingParams

__all__ = ["LLM", "Generation", "SamplingParams", "StepEntry"]


class LLM:
    def __init__(self, model_dir=None, dtype: str = "bfloat16", max_tokens: int = 65536,
                 max_seqs: Optional[int] = None, device: str = "cuda:0", model: Optional[Model] = None):
        """``max_tokens``: the most tokens all live sequences hold together (each rounded
        up to a page of 64); it sizes the cache.  ``model``: a model that exists already
        (then ``model_dir``, ``dtype`` and ``device`` are not used)."""
        if (model is None) == (model_dir is None):
            raise ValueError("LLM needs a model folder or a model, not both")
        self.model = model if model is not None else Model.from_folder(model_dir, dtype=dtype,
                                                                       device=device)
        self.engine = Engine(self.model, max_tokens=max_tokens, max_seqs=max_seqs)
        self.use_graph = True          # replay decode steps from a CUDA graph
        self.last_decode: dict = {}    # wall-clock account of the last call's decode steps

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bfloat16", max_tokens: int = 65536,
               max_seqs: Optional[int] = None, device: str = "cuda:0", storage=None) -> "LLM":
        """Random weights for ``config`` (a config.json dictionary) made in device memory:
        the model that ``synth`` would write for the same configuration and seed, without
        the folder (see ``Model.random``)."""
        return cls(model=Model.random(config, seed, dtype, device, storage), max_tokens=max_tokens,
                   max_seqs=max_seqs)

    @property
    def stop_token_ids(self) -> tuple:
        return tuple(self.model.spec.stop_token_ids)

    def generate(self, prompts: Sequence[Sequence[int]], n: int = 64, temperature: float = 0.7,
                 top_k: int = 40, top_p: float = 0.9, repeat_penalty: float = 1.1, seed: int = 0,
                 stop_ids: Optional[Sequence[int]] = None, ignore_eos: bool = False,
                 ctx: Optional[int] = None, max_batch: int = 64) -> list[Generation]:
        """One ``Generation`` (tokens, finish_reason, stop_token) per prompt, in order.
        Requests that do not fit the cache together run as consecutive batches."""
        if stop_ids is None:
            stop_ids = () if ignore_eos else self.stop_token_ids
        params = SamplingParams(temperature, top_k, top_p, repeat_penalty)
        backend = EngineBackend(self.engine, params, seed, max_context=ctx,
                                use_graph=self.use_graph)
        out = generate(backend, prompts, n, stop_ids, max_batch)
        backend.finish()
        self.last_decode = dict(seconds=backend.decode_seconds, steps=backend.decode_steps,
                                tokens=backend.decode_tokens)
        return out

    def step(self, entries: Sequence[StepEntry]):
        """The step function itself: see ``Engine.step``."""
        return self.engine.step(entries)

    def open_sequence(self):
        return self.engine.open_sequence()

    def close_sequence(self, seq) -> None:
        self.engine.close_sequence(seq)
