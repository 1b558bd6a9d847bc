"""Chooses one token per row of logits on the device."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import kernels
from .params import RECENT_USE, SamplingParams


class Sampler:
    """Holds the device buffers of one sampling call site.  Random numbers come from the
    per-slot records of the cache (``seq_state``), so a sequence's choices depend on the
    seed, its stream id and how many tokens it has drawn: not on the batch."""

    def __init__(self, seq_state: torch.Tensor, device):
        self.seq_state = seq_state
        self.device = torch.device(device)
        self._recent_host: Optional[torch.Tensor] = None
        self._recent_dev: Optional[torch.Tensor] = None
        self._cap = 0

    def seed(self, slots: Sequence[int], streams: Sequence[int], seed: int) -> None:
        s = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        t = torch.tensor(list(streams), dtype=torch.int32, device=self.device)
        kernels.seed_slots(self.seq_state, s, t, int(seed))

    def set_recent(self, slots: Sequence[int], tokens: Sequence[Sequence[int]]) -> None:
        """Starts each slot's ring of recent ids with the last ``RECENT_USE`` of its tokens
        (a prompt's tail); every id sampled with a repeat penalty is added on the device."""
        n = len(slots)
        if n == 0:
            return
        if self._recent_host is None or self._cap < n:
            self._cap = cap = max(n, 64)
            self._recent_host = torch.zeros((cap, RECENT_USE + 1), dtype=torch.int32, pin_memory=True)
            self._recent_dev = torch.zeros((cap, RECENT_USE + 1), dtype=torch.int32, device=self.device)
            self._slots_dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        # the last call's copy out of the staging buffer must be over before it is refilled
        torch.cuda.current_stream().synchronize()
        host = self._recent_host.numpy()
        for r, ids in enumerate(tokens):
            ids = list(ids)[-RECENT_USE:]
            host[r, 0] = len(ids)
            host[r, 1:1 + len(ids)] = ids
        self._recent_dev.copy_(self._recent_host, non_blocking=True)
        self._slots_dev[:n].copy_(torch.tensor(list(slots), dtype=torch.int32))
        kernels.recent_set(self.seq_state, self._slots_dev[:n], self._recent_dev)

    def sample(self, logits: torch.Tensor, params: SamplingParams, slots: torch.Tensor,
               out_ids: torch.Tensor) -> None:
        """logits float32 [R, V] (changed in place by a repeat penalty); slots int32 [R];
        out_ids int32 [R].  The repeat penalty looks at the ids in the sequences' rings
        (``set_recent``) and adds the chosen one to them."""
        if not params.filtered:
            kernels.sample_rows(logits, params.temperature, self.seq_state, slots, out_ids)
            return
        kernels.sample_filtered(logits, params.temperature, params.top_k, params.top_p,
                                params.repeat_penalty, None, None, self.seq_state, slots, out_ids,
                                append=True)
