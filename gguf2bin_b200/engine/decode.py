"""Decoding a fixed batch one token per step without host work in between.

A ``DecodeSession`` is the step function specialised to "every sequence of this batch
goes on by one token, and the token is the one just sampled": the batch's index tensors
stay on the device, the sampler writes each new token where the next step reads it, and
positions advance on the device.  It runs the same model, cache, kernels and sampler as
``Engine.step``; only the bookkeeping differs.

The launches of one such step (the model's forward pass, sampling, the advance) depend on
the step's shape only: how many sequences, how wide their page table, how it samples.
Which sequences, pages, positions and tokens is data on the device.  So the device buffers
of a shape and the CUDA graph captured over them belong to the engine, as a
``DecodeRunner`` kept by shape: a new session of a shape that was seen before (another
call, or the batch that is left when a sequence ends and an earlier batch had that size)
writes its sequences' data into the runner's buffers and replays the graph that is there.
A graph is captured only once a shape has run plainly a few times, and a batch of more than
a few sequences runs with its rows rounded up to a multiple of eight: the rows beyond its
sequences feed the cache's spare page and slot, and nobody reads what they produce.  When a
sequence of the batch ends, its row becomes one more of these and the others stay where they
are (``retire``); only when eight rows fewer will do is the batch put together anew.  So a
batch whose sequences end one after another passes through few shapes, keeps replaying the
graph it has, and loses no step that was launched ahead.

The pages of every sequence must be reserved up to the length it can reach before the
session starts (the page table is uploaded once).

``step`` is the host-facing form (tokens in, sampled tokens out).  It keeps the GPU busy
across the host's turn: as soon as a step's tokens are on their way back it launches the
next step ahead, fed by the tokens just sampled, which is what the caller hands in next in
all but the last step of a sequence.  If the caller then wants something else (other tokens,
other sequences, or nothing more) the step launched ahead is taken back: it wrote the key
and value of a token at a position that is written again or never read, and its bookkeeping
(lengths, positions, draw counters) is rewound.  That only holds for what is stored by
position: a layer that keeps a state of fixed size has folded the token into it for good,
so a model with such a layer never runs ahead.
"""
from __future__ import annotations

import weakref
from typing import Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.pool import Sequence as CacheSequence
from ..cache.storage import KVNeed
from ..parts.base import StepContext
from ..sampling import Sampler, SamplingParams
from .step import Engine, StepError, capture_graph

PAGE_TABLE_STEP = 4          # page-table widths are rounded up to this many pages (one 256-key chunk)
ROW_STEP = 8                 # batches of more than EXACT_ROWS sequences run this many rows at a time
EXACT_ROWS = 4


def padded_rows(n_seqs: int) -> int:
    """Rows that a decode step of ``n_seqs`` sequences runs."""
    return n_seqs if n_seqs <= EXACT_ROWS else -(-n_seqs // ROW_STEP) * ROW_STEP


class DecodeRunner:
    """Device buffers and, in time, the captured graph of decode steps of one shape."""

    EAGER_STEPS = 4          # plain steps of a shape before its graph is captured

    def __init__(self, engine: Engine, batch: int, table_width: int, params: Optional[SamplingParams]):
        self.engine, self.batch, self.table_width = engine, batch, table_width
        self.params = params                    # None: the caller samples after the step, outside a graph
        B, P, dev = batch, table_width, engine.device
        self.n_meta = 4 * B + B * P
        self._meta = torch.zeros(self.n_meta, dtype=torch.int32, device=dev)
        self._meta_host = torch.zeros(self.n_meta, dtype=torch.int32, pin_memory=True)
        self._uploaded = torch.cuda.Event()
        self.tok_ids = self._meta[0:B]
        self.tok_pos = self._meta[B:2 * B]
        self.tok_seq = self._meta[2 * B:3 * B]
        self.slots = self._meta[3 * B:4 * B]
        self.page_table = self._meta[4 * B:].view(B, P)
        self.want_rows = torch.arange(B, dtype=torch.int32, device=dev)
        self.ctx = StepContext(
            n_tokens=B, n_seqs=B, tok_ids=self.tok_ids, tok_pos=self.tok_pos, tok_seq=self.tok_seq,
            page_table=self.page_table, page_size=engine.cache.page_size,
            workspace=engine.workspace, dtype=engine.model.dtype, q_lens=[1] * B,
            past_lens=[0] * B, slots=[0] * B, max_kv_len=P * engine.cache.page_size)
        # what a session needs to talk to the host, kept here so that a new session of a known
        # shape allocates nothing (pinned memory is slow to get)
        self.pinned_in = torch.empty(B, dtype=torch.int32, pin_memory=True)
        self.pinned_out = [torch.empty(B, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.out_ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.out_turn = 0
        self.tokens_uploaded = torch.cuda.Event()
        self._owner = None                      # weak: the session holds the runner, not the other way round
        self.logits: Optional[torch.Tensor] = None
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_generation = -1
        self.plain_steps = 0
        self.launches_per_step = 0

    def bind(self, session: "DecodeSession", keep_tokens: bool = False) -> None:
        """Writes the session's sequences into the buffers, each in its row: positions, slots,
        pages.  The other rows start at position 0 of the cache's spare page with the spare slot's
        record; they advance with the others, so they stay below the positions the table covers.
        ``keep_tokens``: the token ids that the last step left on the device stay (the rows have
        steps behind them)."""
        B, P = self.batch, self.table_width
        cache = self.engine.cache
        self._uploaded.synchronize()               # the staging buffer's last copy is over
        host = self._meta_host.numpy()
        host[:2 * B] = 0
        host[2 * B:3 * B] = np.arange(B)
        host[3 * B:4 * B] = cache.spare_slot
        host[4 * B:] = cache.spare_page
        slots = [cache.spare_slot] * B
        for r, s in zip(session.rows, session.seqs):
            host[B + r] = s.length                 # position of the next token
            host[3 * B + r] = slots[r] = s.slot
            host[4 * B + r * P:4 * B + r * P + len(s.pages)] = s.pages
        first = B if keep_tokens else 0
        self._meta[first:].copy_(self._meta_host[first:], non_blocking=True)
        self._uploaded.record()
        self.ctx.slots = slots
        # the page table is as wide as what is reserved; kernels that size their work by the keys plan with what is there
        self.ctx.kv_len_hint = max(s.length for s in session.seqs) + 1
        self._owner = weakref.ref(session)

    def owned_by(self, session: "DecodeSession") -> bool:
        return self._owner is not None and self._owner() is session

    def _launch(self) -> None:
        eng = self.engine
        self.logits = eng.workspace.buffer("decode.logits", (self.batch, eng.model.vocab), torch.float32)
        eng.model.forward(self.ctx, eng.cache, self.want_rows, self.batch, logits_out=self.logits)
        p = self.params
        if p is not None:
            if p.filtered:        # the repeat penalty reads and extends the sequences' rings of recent ids
                kernels.sample_filtered(self.logits, p.temperature, p.top_k, p.top_p, p.repeat_penalty,
                                        None, None, eng.cache.seq_state, self.slots, self.tok_ids, append=True)
            else:
                kernels.sample_rows(self.logits, p.temperature, eng.cache.seq_state, self.slots,
                                    self.tok_ids)
            kernels.advance_positions(self.tok_pos, self.batch)

    def run(self, use_graph: bool, eager_steps: int) -> None:
        ws = self.engine.workspace
        if self._graph is not None and ws.generation != self._graph_generation:
            self._graph, self.plain_steps = None, 0           # scratch buffers moved: capture again
        if self._graph is not None and use_graph:
            self._graph.replay()
            return
        before = kernels.launch_count()
        if use_graph and self.plain_steps >= eager_steps:
            torch.cuda.current_stream().synchronize()
            generation = ws.generation
            g, _ = capture_graph(self._launch)
            self.launches_per_step = kernels.launch_count() - before
            self.engine.decode_graph_captures += 1
            if ws.generation == generation:
                self._graph, self._graph_generation = g, generation
                g.replay()
                return
            before = kernels.launch_count()        # a buffer appeared during the capture: run plainly
        self._launch()
        self.launches_per_step = kernels.launch_count() - before
        self.plain_steps += 1


def decode_runner(engine: Engine, batch: int, pages: int, params: Optional[SamplingParams]) -> DecodeRunner:
    """The engine's runner for steps of ``batch`` rows and this way of sampling, made at its first
    use; the least recently used ones go when there are more than ``Engine.DECODE_RUNNERS_KEPT``."""
    width = -(-max(int(pages), 1) // PAGE_TABLE_STEP) * PAGE_TABLE_STEP
    key = (batch, width, params)
    runners = engine.decode_runners
    runner = runners.get(key)
    if runner is None:
        runner = runners[key] = DecodeRunner(engine, batch, width, params)
        while len(runners) > engine.DECODE_RUNNERS_KEPT:
            runners.popitem(last=False)
    else:
        runners.move_to_end(key)
    return runner


class DecodeSession:
    CHECK_EVERY = 64         # collections between two reads of the kernels' status word

    def __init__(self, engine: Engine, seqs: Sequence[CacheSequence], sampler: Sampler,
                 params: SamplingParams, use_graph: bool = True, eager_steps: Optional[int] = None):
        """``eager_steps``: plain steps of this shape before its graph is captured (default:
        ``DecodeRunner.EAGER_STEPS``; at least one, which sizes every scratch buffer)."""
        self.engine, self.seqs, self.sampler, self.params = engine, list(seqs), sampler, params
        B = len(self.seqs)
        self.rows = list(range(B))          # the row of each sequence: they stay where they are when others end
        if B == 0:
            raise StepError("a decode session needs at least one sequence")
        if sampler.seq_state is not engine.cache.seq_state:
            raise StepError("the sampler of a decode session must use the engine's per-slot records")
        # sampling runs inside the step (and its graph): it needs no host data, the recent ids
        # that a repeat penalty looks at are in the sequences' records on the device
        self._sample_in_graph = True
        self.runner = decode_runner(engine, padded_rows(B), max(len(s.pages) for s in self.seqs), params)
        self.runner.bind(self)
        self.use_graph = use_graph and engine.model.graph_safe
        self.eager_steps = max(1, DecodeRunner.EAGER_STEPS if eager_steps is None else int(eager_steps))
        # a step launched ahead can be taken back only if all it stored is stored by position
        self._may_run_ahead = self._sample_in_graph and all(
            isinstance(g["need"], KVNeed) for g in engine.cache.groups.values())
        self._ahead: Optional[list] = None      # tokens, row by row, fed to the step launched ahead, if any
        self._since_check = 0

    def retire(self, seq: CacheSequence) -> bool:
        """A sequence of the batch has ended.  Its row goes on as one more row of padding (spare
        page, spare slot) and the others stay in their rows, so the shape, its graph and a step
        launched ahead (whose other rows are what they would have been) all live on.  False: the
        batch is better rebuilt without the sequence, because fewer rows will do, and the session
        must not be used further."""
        k = next((k for k, s in enumerate(self.seqs) if s is seq), None)
        if k is None:
            return True
        if padded_rows(len(self.seqs) - 1) < self.runner.batch or not self.runner.owned_by(self):
            return False
        del self.seqs[k], self.rows[k]
        self.runner.bind(self, keep_tokens=True)
        return True

    @property
    def batch(self) -> int:
        return len(self.seqs)

    @property
    def logits(self) -> torch.Tensor:
        """The last step's logits, float32 [batch, vocab] (scratch: valid until the next step)."""
        if self.rows == list(range(self.batch)):
            return self.runner.logits[:self.batch]
        return self.runner.logits[self.rows]

    @property
    def launches_per_step(self) -> int:
        return self.runner.launches_per_step

    def _own_runner(self) -> None:
        """Another session of the same shape may have used the runner since: write this
        session's data back (positions follow from the sequences' lengths)."""
        if not self.runner.owned_by(self):
            self.runner.bind(self)

    def set_tokens(self, tokens: Sequence[int]) -> None:
        """The tokens the next step feeds (host to device, from pinned memory)."""
        self._own_runner()
        runner = self.runner
        runner.tokens_uploaded.synchronize()       # the staging buffer's last copy is over
        staged = runner.pinned_in.numpy()
        staged[:] = 0
        staged[self.rows] = tokens
        runner.tok_ids.copy_(runner.pinned_in, non_blocking=True)
        runner.tokens_uploaded.record()

    def run(self) -> None:
        """One step: feeds ``tok_ids``, leaves the sampled tokens in ``tok_ids`` and the
        logits in ``logits``."""
        page = self.engine.cache.page_size
        if any(s.length + 1 > len(s.pages) * page for s in self.seqs):
            raise StepError("a sequence of the decode session has no reserved page left")
        self._own_runner()
        runner = self.runner
        past = [0] * runner.batch
        for r, s in zip(self.rows, self.seqs):
            past[r] = s.length
        runner.ctx.past_lens = past
        runner.run(self.use_graph, self.eager_steps)
        if not self._sample_in_graph:
            self.sampler.sample(runner.logits, self.params, runner.slots, runner.tok_ids)
            kernels.advance_positions(runner.tok_pos, runner.batch)
        for s in self.seqs:
            s.length += 1

    def read_tokens(self) -> list:
        """The tokens sampled by the last step (device to host)."""
        by_row = self._collect(self._send_back())
        return [by_row[r] for r in self.rows]

    def _send_back(self) -> int:
        """Starts the copy of the last step's tokens to the host; returns its turn."""
        runner = self.runner
        turn = runner.out_turn
        runner.out_turn ^= 1
        runner.pinned_out[turn].copy_(runner.tok_ids, non_blocking=True)
        runner.out_ready[turn].record()
        return turn

    def _collect(self, turn: int) -> list:
        """The tokens of that copy, row by row."""
        self.runner.out_ready[turn].synchronize()
        self._since_check += 1
        if self._since_check >= self.CHECK_EVERY:
            self.check()
        return self.runner.pinned_out[turn].tolist()

    def check(self) -> None:
        """Reports a kernel that gave up a bounded wait (see ``Engine.check``).  Reading the
        word costs a small copy, so steps do it every ``CHECK_EVERY`` collections; the session's
        owner calls it once more before it hands tokens on for good."""
        self._since_check = 0
        self.engine.check()

    def _room_for_one_more(self) -> bool:
        page = self.engine.cache.page_size
        limit = self.engine.model.spec.max_positions
        return all(s.length + 1 <= len(s.pages) * page and s.length + 1 <= limit for s in self.seqs)

    def step(self, tokens: Sequence[int]) -> list:
        """Feeds one token per sequence and returns the sampled next tokens, through pinned
        host memory both ways.  Steps that sample on the device are launched one ahead."""
        tokens = [int(t) for t in tokens]
        if self._ahead is not None and tokens == [self._ahead[r] for r in self.rows]:
            turn = self._ahead_turn                  # the step launched ahead is this one
        else:
            self.take_back()
            self.set_tokens(tokens)
            self.run()
            turn = self._send_back()
        self._ahead = None
        ahead_turn = None
        if self._may_run_ahead and self._room_for_one_more():
            self.run()                               # the next step, fed by the tokens being sampled now;
            ahead_turn = self._send_back()           # queued before this step's tokens are waited for
        by_row = self._collect(turn)
        if ahead_turn is not None:
            self._ahead, self._ahead_turn = by_row, ahead_turn
        return [by_row[r] for r in self.rows]

    def take_back(self) -> None:
        """Undoes a step launched ahead that nobody asked for."""
        if self._ahead is None:
            return
        self._ahead = None
        self._own_runner()
        kernels.rewind_step(self.runner.tok_pos, self.runner.batch, self.sampler.seq_state, self.runner.slots,
                            self.params.temperature > 0.0, self.params.filtered)
        for s in self.seqs:
            s.length -= 1
