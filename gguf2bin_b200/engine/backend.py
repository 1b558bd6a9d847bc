"""The generation loop's backend on the device: the engine's step function plus the
sampler, one call per step, host tokens in and sampled tokens out."""
from __future__ import annotations

import time
from typing import Optional, Sequence

import torch

from ..cache.pool import Sequence as CacheSequence
from ..sampling import RECENT_USE, Sampler, SamplingParams
from .decode import DecodeSession
from .step import Engine, StepEntry, StepError


class _Handle:
    __slots__ = ("seq",)

    def __init__(self, seq: CacheSequence):
        self.seq = seq


class EngineBackend:
    def __init__(self, engine: Engine, params: SamplingParams, seed: int = 0,
                 max_context: Optional[int] = None, use_graph: bool = True):
        self.engine = engine
        self.params = params
        self.seed = int(seed)
        self.sampler = Sampler(engine.cache.seq_state, engine.device)
        limit = engine.model.spec.max_positions
        self.max_context = min(limit, int(max_context)) if max_context else limit
        self.page_size = engine.cache.page_size
        self._ids = torch.empty(1024, dtype=torch.int32, device=engine.device)
        self._slots = torch.empty(1024, dtype=torch.int32, device=engine.device)
        self.use_graph = use_graph
        self._session: Optional[DecodeSession] = None
        # wall-clock account of the decode calls, for measurements through this API
        self.decode_seconds = 0.0
        self.decode_steps = 0
        self.decode_tokens = 0

    @property
    def free_pages(self) -> int:
        return self.engine.cache.table.pages.n_free

    def open(self, stream_id: int, reserve_tokens: int) -> _Handle:
        seq = self.engine.open_sequence()
        try:
            self.engine.cache.reserve(seq, reserve_tokens)
        except Exception:
            self.engine.close_sequence(seq)
            raise
        self.sampler.seed([seq.slot], [stream_id], self.seed)
        return _Handle(seq)

    def _drop_session(self) -> None:
        """Ends the decode session (a step it launched ahead is taken back first)."""
        if self._session is not None:
            self._session.take_back()
            self._session = None

    def finish(self) -> None:
        """Called once the caller is about to hand the generated tokens on: ends the decode
        session and reports a kernel that gave up a wait in any step since the last check."""
        self._drop_session()
        self.engine.check()

    def close(self, handle: _Handle) -> None:
        if handle.seq.slot >= 0:
            if self._session is not None and not self._session.retire(handle.seq):
                self._drop_session()           # the others are better off as a batch of their own
            self.engine.close_sequence(handle.seq)

    def _sample(self, logits: torch.Tensor, handles: Sequence[_Handle]) -> list:
        R = len(handles)
        if self._ids.shape[0] < R:
            self._ids = torch.empty(2 * R, dtype=torch.int32, device=self.engine.device)
            self._slots = torch.empty(2 * R, dtype=torch.int32, device=self.engine.device)
        self._slots[:R].copy_(torch.tensor([h.seq.slot for h in handles], dtype=torch.int32))
        self.sampler.sample(logits, self.params, self._slots[:R], self._ids[:R])
        out = self._ids[:R].tolist()
        self.engine.check()                    # never hand on tokens of a launch that gave up a wait
        return out

    def prefill(self, handles: Sequence[_Handle], prompts: Sequence[Sequence[int]]) -> list:
        self._drop_session()
        entries = [StepEntry(h.seq, p, (len(p) - 1,)) for h, p in zip(handles, prompts)]
        logits = self.engine.step(entries)
        if self.params.repeat_penalty != 1.0:  # the tails of the prompts: what the penalty looks back over first
            self.sampler.set_recent([h.seq.slot for h in handles], [p[-RECENT_USE:] for p in prompts])
        return self._sample(logits, handles)

    def decode(self, handles: Sequence[_Handle], tokens: Sequence[int]) -> list:
        """Feeds one token per sequence (host to device), returns the sampled next tokens
        (device to host).  While the same sequences keep decoding, the step runs as a
        ``DecodeSession`` (index tensors resident, launches replayed from a graph).  With a repeat
        penalty the tokens fed are expected to be the ones sampled: the recent ids that the penalty
        reads are kept on the device as they are sampled."""
        t0 = time.perf_counter()
        V = self.engine.model.vocab
        for t in tokens:
            if not (0 <= int(t) < V):
                raise StepError(f"token id {t} outside the vocabulary 0..{V - 1}")
        session = self._session
        if session is None or len(session.seqs) != len(handles) or any(
                s is not h.seq for s, h in zip(session.seqs, handles)):
            self._drop_session()
            session = self._session = DecodeSession(self.engine, [h.seq for h in handles], self.sampler,
                                                    self.params, self.use_graph)
        out = session.step(tokens)
        self.decode_seconds += time.perf_counter() - t0
        self.decode_steps += 1
        self.decode_tokens += len(handles)
        return out
