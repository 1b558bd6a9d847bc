"""The step function: a batch of sequences, their next tokens, the cache, the logits at
the wanted places.

A step runs only the tokens it is given, as one ragged batch: the tokens of all
sequences one after another, each token with its own absolute position; no sequence is
padded to another's length.  Rows that fill a step up to a round number of rows (so that
steps of other lengths find the same launches) are the tokens of a sequence of their own
on the cache's spare page: no result of the others depends on them.  Sequences of a step
may be at any position: all prompts at once, then one token each, or a prompt cut into
pieces.

Before anything is launched the whole step is checked on the host (token ids, room in
the cache, positions); a refused step changes nothing.
"""
from __future__ import annotations

import gc
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Optional, Sequence as Seq

import numpy as np
import torch

from ..cache.pool import CacheError, Sequence
from ..cache.storage import Cache
from ..parts.base import ATTN_TILE_ROWS, ATTN_WIDE_TILE_ROWS, StepContext
from .model import Model
from .workspace import Workspace

SINGLE_TABLE_STEP = 4        # page-table widths of one-token steps are rounded up to this many pages


class StepError(ValueError):
    """A step that cannot run; nothing was changed."""


def capture_graph(launch):
    """Captures what ``launch()`` puts on the current stream in a new CUDA graph; returns the
    graph and ``launch``'s result.  The collector of reference cycles is held off meanwhile: it
    could free an older graph in the middle of the capture, and releasing a graph is an
    operation that a capturing stream forbids (the capture would be lost)."""
    graph = torch.cuda.CUDAGraph()
    collecting = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            result = launch()
    finally:
        if collecting:
            gc.enable()
    return graph, result


@dataclass
class StepEntry:
    """One sequence's share of a step: its next tokens and the indices among them whose
    logits are wanted."""
    seq: Sequence
    tokens: Seq[int]
    want: Seq[int] = field(default_factory=tuple)


class _PaddingSequence:
    """What stands in for a sequence in the rows that fill a prompt step up to a multiple of
    ``PROMPT_ROW_STEP``: the cache's spare slot and spare page, nothing before it."""

    def __init__(self, cache: Cache):
        self.slot, self.pages, self.length = cache.spare_slot, [cache.spare_page], 0


class Engine:
    """A model with its cache and scratch memory; ``step`` is the one way tokens run.

    A step's launches depend on the step's shape only (how many tokens each sequence brings,
    where it stands, how many places are wanted); which tokens, pages and places is data that
    the kernels read from the step's metadata on the device.  So when a shape comes back, the
    launches of its forward pass are captured once in a CUDA graph and replayed from then on:
    a prompt step is a few hundred launches, and the host's share of it (a few microseconds
    each) otherwise competes with the device's.  So that prompts of other lengths find a graph
    too, a prompt step's rows are filled up to a multiple of ``PROMPT_ROW_STEP`` with the tokens of
    a padding sequence on the cache's spare page: what the launches depend on is then the number
    of rows, of sequences, of attention tiles and of wanted places and the width of the page
    table, and prompts of 449 to 512 tokens, say, share one graph."""

    PROMPT_ROW_STEP = 64         # at most one page of padding tokens (the cache has one spare page)

    GRAPH_MIN_TOKENS = 2         # every step that is not one token per sequence (those have their own graphs)
    GRAPHS_KEPT = 64             # one per 64-token bucket of prompt lengths up to 4,096; a graph holds launches, no buffers
    DECODE_RUNNERS_KEPT = 24     # shapes of decode steps whose buffers and graphs are kept (engine/decode.py)

    def __init__(self, model: Model, max_tokens: int, max_seqs: Optional[int] = None,
                 step_graphs: bool = True):
        self.model = model
        self.cache: Cache = model.new_cache(max_tokens, max_seqs)
        self.workspace = Workspace(model.device)
        self.device = model.device
        self._meta_cap = 0
        self._meta_dev: Optional[torch.Tensor] = None
        self._meta_host: Optional[torch.Tensor] = None
        self.step_graphs = step_graphs and model.graph_safe
        self._graphs: "OrderedDict[tuple, tuple]" = OrderedDict()    # shape -> (graph, generation, logits)
        self._seen: "OrderedDict[tuple, int]" = OrderedDict()        # shapes run plainly so far
        self.decode_runners: "OrderedDict[tuple, object]" = OrderedDict()
        self._padding = _PaddingSequence(self.cache)
        self.step_graph_captures = 0       # CUDA graphs captured so far: of prompt-step shapes,
        self.decode_graph_captures = 0     # and of decode shapes (engine/decode.py)

    # ---- sequences -----------------------------------------------------------
    def open_sequence(self) -> Sequence:
        return self.cache.open_sequence()

    def close_sequence(self, seq: Sequence) -> None:
        self.cache.close_sequence(seq)

    @property
    def graph_captures(self) -> int:
        return self.step_graph_captures + self.decode_graph_captures

    def check(self) -> None:
        """Raises ``KernelError`` if a kernel launched so far reported that one of its bounded
        waits gave up (its output is then invalid).  Reads a word from the device, so it waits
        for the stream; callers that are about to read logits or tokens on the host call it
        where they synchronise anyway."""
        if self.model.dtype == torch.bfloat16:
            from .. import kernels_bf16
            kernels_bf16.check_status()

    # ---- step ------------------------------------------------------------------
    def _check(self, entries: Seq[StepEntry]) -> None:
        if not entries:
            raise StepError("a step needs at least one sequence")
        V, maxpos = self.model.vocab, self.model.spec.max_positions
        seen = set()
        for e in entries:
            if e.seq.slot < 0 or self.cache.table.live.get(e.seq.slot) is not e.seq:
                raise StepError("a sequence of the step is not live in this engine's cache")
            if e.seq.slot in seen:
                raise StepError(f"slot {e.seq.slot} appears twice in one step")
            seen.add(e.seq.slot)
            n = len(e.tokens)
            if n < 1:
                raise StepError("every sequence of a step needs at least one token")
            for t in e.tokens:
                if not (0 <= int(t) < V):
                    raise StepError(f"token id {t} outside the vocabulary 0..{V - 1}")
            if e.seq.length + n > maxpos:
                raise StepError(f"sequence would reach {e.seq.length + n} positions; the model "
                                f"allows {maxpos}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"wanted place {w} outside the step's {n} tokens")
        need = sum(self.cache.table.pages_needed(e.seq, e.seq.length + len(e.tokens))
                   for e in entries)
        if need > self.cache.table.pages.n_free:
            raise StepError(f"the cache is full: the step needs {need} more pages of "
                            f"{self.cache.page_size} tokens, {self.cache.table.pages.n_free} free")

    def build_context(self, entries: Seq[StepEntry]) -> tuple[StepContext, torch.Tensor, int]:
        """Host metadata of the step packed into one pinned buffer and copied once."""
        B = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        past = [e.seq.length for e in entries]
        T = sum(q_lens)
        P = max(len(e.seq.pages) for e in entries)
        if T == B:                   # one token each: the table's width in steps, so that the shape's graph lasts
            P = -(-P // SINGLE_TABLE_STEP) * SINGLE_TABLE_STEP
        n_want = sum(len(e.want) for e in entries)
        # prompt-attention work list: tiles of 64 query rows, the longest key ranges first
        tiles, wide = [], []
        t0 = 0
        for b, e in enumerate(entries):
            for r in range(0, q_lens[b], ATTN_TILE_ROWS):
                tiles.append((b, t0 + r, min(ATTN_TILE_ROWS, q_lens[b] - r), past[b] + r))
            for r in range(0, q_lens[b], ATTN_WIDE_TILE_ROWS):
                wide.append((b, t0 + r, min(ATTN_WIDE_TILE_ROWS, q_lens[b] - r), past[b] + r))
            t0 += q_lens[b]
        tiles.sort(key=lambda t: -(t[3] + t[2]))
        wide.sort(key=lambda t: -(t[3] + t[2]))
        n_narrow = len(tiles)
        tiles = tiles + wide
        n_tiles = len(tiles)
        # layout: tiles[n_tiles*4] tok_ids[T] tok_pos[T] tok_seq[T] want[n_want] seq_meta[B*4]
        #         page_table[B*P]   (the tiles come first: the kernel reads them 16 bytes at a time)
        total = 4 * n_tiles + 3 * T + n_want + 4 * B + B * P
        if total > self._meta_cap:
            self._meta_cap = max(2 * total, 1024)
            self._meta_dev = torch.empty(self._meta_cap, dtype=torch.int32, device=self.device)
            self._meta_host = torch.empty(self._meta_cap, dtype=torch.int32, pin_memory=True)
        host = self._meta_host.numpy()
        o_ids = 4 * n_tiles
        o_pos, o_seq, o_want = o_ids + T, o_ids + 2 * T, o_ids + 3 * T
        o_meta = o_want + n_want
        host[:4 * n_tiles] = np.asarray(tiles, dtype=np.int32).reshape(-1)
        o_pt = o_meta + 4 * B
        t0 = w0 = 0
        for b, e in enumerate(entries):
            n = q_lens[b]
            host[o_ids + t0:o_ids + t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            host[o_pos + t0:o_pos + t0 + n] = np.arange(past[b], past[b] + n, dtype=np.int32)
            host[o_seq + t0:o_seq + t0 + n] = b
            for w in e.want:
                host[o_want + w0] = t0 + int(w)
                w0 += 1
            host[o_meta + 4 * b:o_meta + 4 * b + 4] = (t0, n, past[b], e.seq.slot)
            row = host[o_pt + b * P:o_pt + (b + 1) * P]
            row[:len(e.seq.pages)] = e.seq.pages
            row[len(e.seq.pages):] = 0
            t0 += n
        dev = self._meta_dev
        dev[:total].copy_(self._meta_host[:total], non_blocking=True)
        ctx = StepContext(
            n_tokens=T, n_seqs=B, tok_ids=dev[o_ids:o_ids + T], tok_pos=dev[o_pos:o_pos + T],
            tok_seq=dev[o_seq:o_seq + T], page_table=dev[o_pt:o_pt + B * P].view(B, P),
            page_size=self.cache.page_size, workspace=self.workspace, dtype=self.model.dtype,
            q_lens=q_lens, past_lens=past, slots=[e.seq.slot for e in entries],
            max_kv_len=max(p + n for p, n in zip(past, q_lens)),
            seq_meta=dev[o_meta:o_meta + 4 * B].view(B, 4),
            attn_tiles=dev[:4 * n_narrow].view(n_narrow, 4), n_attn_tiles=n_narrow,
            attn_tiles_wide=dev[4 * n_narrow:4 * n_tiles].view(n_tiles - n_narrow, 4),
            n_attn_tiles_wide=n_tiles - n_narrow)
        return ctx, dev[o_want:o_want + n_want], n_want

    def step(self, entries: Seq[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the entries' tokens as one batch.  Returns float32 logits
        [number of wanted places, vocab] in the order of the entries and of their
        ``want`` (None when nothing is wanted).  The tensor is scratch memory: it is
        valid until the next step."""
        self._check(entries)
        for e in entries:
            self.cache.reserve(e.seq, e.seq.length + len(e.tokens))
        # the pinned staging buffer is reused: the previous step's copy must be over
        torch.cuda.current_stream().synchronize()
        self.check()                 # a kernel of an earlier step that gave up a wait is reported here
        run = self._filled_up(entries)
        ctx, want_rows, n_want = self.build_context(run)
        logits = self._forward(run, ctx, want_rows, n_want)
        for e in entries:
            e.seq.length += len(e.tokens)
        return logits

    def _filled_up(self, entries: Seq[StepEntry]) -> Seq[StepEntry]:
        """The step's entries, with a last one of padding tokens when the step is one that graphs are
        kept for (any step that is not one token per sequence) and its rows are no multiple
        of ``PROMPT_ROW_STEP``.  The padding's rows are rows of a sequence of their own (nothing of
        the others' results depends on them); its keys and values land on the spare page."""
        T = sum(len(e.tokens) for e in entries)
        if not self.step_graphs or T == len(entries) or T < self.GRAPH_MIN_TOKENS:
            return entries
        fill = -T % self.PROMPT_ROW_STEP
        if fill == 0:
            return entries
        return list(entries) + [StepEntry(self._padding, [0] * fill, ())]

    def _forward(self, entries, ctx: StepContext, want_rows, n_want) -> Optional[torch.Tensor]:
        """The model's forward pass of this step: replayed from a graph when the step's shape
        has been captured, captured at its second appearance (one token per sequence) or its third
        (prompts), run plainly otherwise."""
        single = ctx.all_single
        if single:
            # One token per sequence: the kernels take every position from device memory, so one
            # graph serves the shape for as long as the page table keeps its width; the attention
            # is laid out for all the keys the table covers and plans with those there are.
            ctx.kv_len_hint = ctx.max_kv_len
            ctx.max_kv_len = ctx.page_table.shape[1] * self.cache.page_size
        if not self.step_graphs or (ctx.n_tokens < self.GRAPH_MIN_TOKENS and not single):
            return self.model.forward(ctx, self.cache, want_rows, n_want)
        # everything a launch argument or a buffer address is derived from
        if single:
            key = ("single", ctx.n_seqs, tuple(len(e.want) for e in entries), ctx.page_table.shape[1],
                   self._meta_dev.data_ptr())
        else:
            # which tokens, positions, pages, tiles and places is data on the device; the launches see
            # only how many there are (the same numbers fix where each table lies in the step's metadata)
            key = ("prompt", ctx.n_tokens, ctx.n_seqs, ctx.n_attn_tiles, ctx.n_attn_tiles_wide, n_want,
                   ctx.page_table.shape[1], self._meta_dev.data_ptr())
        hit = self._graphs.get(key)
        if hit is not None:
            graph, generation, logits = hit
            if generation == self.workspace.generation:
                self._graphs.move_to_end(key)
                graph.replay()
                return logits
            del self._graphs[key]                     # scratch buffers moved since the capture
        if self._seen.get(key, 0) >= (1 if single else 2):
            # The shape ran plainly before, so every scratch buffer it needs exists already.  A prompt
            # shape is captured when it comes for the third time: a capture costs as much as two or three
            # plain steps, and of the shapes of ragged batches most never come back.
            torch.cuda.current_stream().synchronize()
            generation = self.workspace.generation
            graph, logits = capture_graph(lambda: self.model.forward(ctx, self.cache, want_rows, n_want))
            self.step_graph_captures += 1
            if self.workspace.generation == generation:
                self._graphs[key] = (graph, generation, logits)
                while len(self._graphs) > self.GRAPHS_KEPT:
                    self._graphs.popitem(last=False)
                graph.replay()
                return logits
            # a buffer was created during the capture after all: run plainly, try again next time
        self._seen[key] = self._seen.get(key, 0) + 1
        while len(self._seen) > 256:
            self._seen.popitem(last=False)
        return self.model.forward(ctx, self.cache, want_rows, n_want)
