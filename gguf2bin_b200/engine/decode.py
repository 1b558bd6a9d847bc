"""Decoding a fixed batch one token per step without host work in between.

A ``DecodeSession`` is the step function specialised to "every sequence of this batch
goes on by one token, and the token is the one just sampled": the batch's index tensors
stay on the device, the sampler writes each new token where the next step reads it, and
positions advance on the device.  The launches of one step (the model's forward pass,
sampling, the advance) are the same every time, so after two plain steps they are
captured once in a CUDA graph and replayed.  It runs the same model, cache, kernels and
sampler as ``Engine.step``; only the bookkeeping differs.

The pages of every sequence must be reserved up to the length it can reach before the
session starts (the page table is uploaded once).

``step`` is the host-facing form (tokens in, sampled tokens out).  It keeps the GPU busy
across the host's turn: as soon as a step's tokens are on their way back it launches the
next step ahead, fed by the tokens just sampled, which is what the caller hands in next in
all but the last step of a sequence.  If the caller then wants something else (other tokens,
other sequences, or nothing more) the step launched ahead is taken back: it wrote the key
and value of a token at a position that is written again or never read, and its bookkeeping
(lengths, positions, draw counters) is rewound.
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.pool import Sequence as CacheSequence
from ..parts.base import StepContext
from ..sampling import Sampler, SamplingParams
from .step import Engine, StepError


class DecodeSession:
    EAGER_STEPS = 1          # plain steps before the graph is captured (the first sizes every buffer)

    def __init__(self, engine: Engine, seqs: Sequence[CacheSequence], sampler: Sampler,
                 params: SamplingParams, use_graph: bool = True):
        self.engine, self.seqs, self.sampler, self.params = engine, list(seqs), sampler, params
        B = len(self.seqs)
        if B == 0:
            raise StepError("a decode session needs at least one sequence")
        dev = engine.device
        P = max(len(s.pages) for s in self.seqs)
        host = np.zeros(3 * B + B * P, dtype=np.int32)
        host[B:2 * B] = [s.length for s in self.seqs]            # positions of the next tokens
        host[2 * B:3 * B] = np.arange(B)
        for b, s in enumerate(self.seqs):
            host[3 * B + b * P:3 * B + b * P + len(s.pages)] = s.pages
        self._meta = torch.from_numpy(host).to(dev)
        self.tok_ids = self._meta[0:B]
        self.tok_pos = self._meta[B:2 * B]
        self.tok_seq = self._meta[2 * B:3 * B]
        self.page_table = self._meta[3 * B:].view(B, P)
        self.slots = torch.tensor([s.slot for s in self.seqs], dtype=torch.int32, device=dev)
        self.want_rows = torch.arange(B, dtype=torch.int32, device=dev)
        self.logits = torch.empty(B, engine.model.vocab, dtype=torch.float32, device=dev)
        self._pinned_in = torch.empty(B, dtype=torch.int32, pin_memory=True)
        self._pinned_out = [torch.empty(B, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._out_ready = [torch.cuda.Event(), torch.cuda.Event()]
        self._out_turn = 0
        self._ahead: Optional[list] = None      # tokens fed to the step launched ahead, if any
        self.ctx = StepContext(
            n_tokens=B, n_seqs=B, tok_ids=self.tok_ids, tok_pos=self.tok_pos, tok_seq=self.tok_seq,
            page_table=self.page_table, page_size=engine.cache.page_size,
            workspace=engine.workspace, dtype=engine.model.dtype, q_lens=[1] * B,
            past_lens=[s.length for s in self.seqs], slots=[s.slot for s in self.seqs],
            max_kv_len=max(len(s.pages) for s in self.seqs) * engine.cache.page_size)
        self.use_graph = use_graph and engine.model.graph_safe
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_generation = -1
        self._steps = 0
        self.launches_per_step = 0
        # sampling inside the graph needs no host data; filtered sampling uploads the
        # recent tokens every step and therefore runs after the graph
        self._sample_in_graph = not params.filtered

    @property
    def batch(self) -> int:
        return len(self.seqs)

    def set_tokens(self, tokens: Sequence[int]) -> None:
        """The tokens the next step feeds (host to device, from pinned memory)."""
        self._pinned_in.copy_(torch.tensor(list(tokens), dtype=torch.int32))
        self.tok_ids.copy_(self._pinned_in, non_blocking=True)

    def _launch(self) -> None:
        self.engine.model.forward(self.ctx, self.engine.cache, self.want_rows, self.batch,
                                  logits_out=self.logits)
        if self._sample_in_graph:
            kernels.sample_rows(self.logits, self.params.temperature, self.sampler.seq_state,
                                self.slots, self.tok_ids)
            kernels.advance_positions(self.tok_pos, self.batch)

    def run(self, recent=None) -> None:
        """One step: feeds ``tok_ids``, leaves the sampled tokens in ``tok_ids`` and the
        logits in ``logits``."""
        page = self.engine.cache.page_size
        if any(s.length + 1 > len(s.pages) * page for s in self.seqs):
            raise StepError("a sequence of the decode session has no reserved page left")
        ws = self.engine.workspace
        if self._graph is not None and ws.generation != self._graph_generation:
            self._graph, self._steps = None, 0        # scratch buffers moved: capture again
        if self._graph is not None:
            self._graph.replay()
        elif self.use_graph and self._steps >= self.EAGER_STEPS:
            torch.cuda.current_stream().synchronize()
            before = kernels.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._launch()
            self.launches_per_step = kernels.launch_count() - before
            self._graph, self._graph_generation = g, ws.generation
            g.replay()
        else:
            before = kernels.launch_count()
            self._launch()
            self.launches_per_step = kernels.launch_count() - before
        if not self._sample_in_graph:
            self.sampler.sample(self.logits, self.params, self.slots, self.tok_ids, recent)
            kernels.advance_positions(self.tok_pos, self.batch)
        for s in self.seqs:
            s.length += 1
        self._steps += 1

    def read_tokens(self) -> list:
        """The tokens sampled by the last step (device to host)."""
        return self._collect(self._send_back())

    def _send_back(self) -> int:
        """Starts the copy of the last step's tokens to the host; returns its turn."""
        turn = self._out_turn
        self._out_turn ^= 1
        self._pinned_out[turn].copy_(self.tok_ids, non_blocking=True)
        self._out_ready[turn].record()
        return turn

    def _collect(self, turn: int) -> list:
        self._out_ready[turn].synchronize()
        return self._pinned_out[turn].tolist()

    def _room_for_one_more(self) -> bool:
        page = self.engine.cache.page_size
        limit = self.engine.model.spec.max_positions
        return all(s.length + 1 <= len(s.pages) * page and s.length + 1 <= limit for s in self.seqs)

    def step(self, tokens: Sequence[int], recent=None) -> list:
        """Feeds one token per sequence and returns the sampled next tokens, through pinned
        host memory both ways.  Steps that sample on the device are launched one ahead."""
        tokens = [int(t) for t in tokens]
        if self._ahead is not None and tokens == self._ahead:
            turn = self._ahead_turn                  # the step launched ahead is this one
        else:
            self.take_back()
            self.set_tokens(tokens)
            self.run(recent)
            turn = self._send_back()
        self._ahead = None
        ahead_turn = None
        if self._sample_in_graph and self._room_for_one_more():
            self.run(None)                           # the next step, fed by the tokens being sampled now;
            ahead_turn = self._send_back()           # queued before this step's tokens are waited for
        out = self._collect(turn)
        if ahead_turn is not None:
            self._ahead, self._ahead_turn = out, ahead_turn
        return out

    def take_back(self) -> None:
        """Undoes a step launched ahead that nobody asked for."""
        if self._ahead is None:
            return
        self._ahead = None
        kernels.rewind_step(self.tok_pos, self.batch, self.sampler.seq_state, self.slots,
                            self.params.temperature > 0.0)
        for s in self.seqs:
            s.length -= 1
