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

    def sample(self, logits: torch.Tensor, params: SamplingParams, slots: torch.Tensor,
               out_ids: torch.Tensor, recent: Optional[Sequence[Sequence[int]]] = None) -> None:
        """logits float32 [R, V] (changed in place by a repeat penalty); slots int32 [R];
        out_ids int32 [R].  ``recent``: each row's last tokens, oldest first."""
        if not params.filtered:
            kernels.sample_rows(logits, params.temperature, self.seq_state, slots, out_ids)
            return
        R = logits.shape[0]
        if self._recent_host is None or self._cap < R:
            # ids [cap, RECENT_USE] and counts [cap], each contiguous, in one staging buffer
            self._cap = cap = max(R, 64)
            self._recent_host = torch.zeros(cap * (RECENT_USE + 1), dtype=torch.int32, pin_memory=True)
            self._recent_dev = torch.zeros(cap * (RECENT_USE + 1), dtype=torch.int32, device=self.device)
        cap = self._cap
        # the last call's copy out of the staging buffer must be over before it is refilled
        torch.cuda.current_stream().synchronize()
        host_ids = self._recent_host[:cap * RECENT_USE].view(cap, RECENT_USE)
        host_n = self._recent_host[cap * RECENT_USE:]
        for r in range(R):
            ids = list(recent[r])[-RECENT_USE:] if recent is not None else []
            host_n[r] = len(ids)
            if ids:
                host_ids[r, :len(ids)] = torch.tensor(ids, dtype=torch.int32)
        self._recent_dev.copy_(self._recent_host, non_blocking=True)
        dev_ids = self._recent_dev[:cap * RECENT_USE].view(cap, RECENT_USE)
        dev_n = self._recent_dev[cap * RECENT_USE:]
        kernels.sample_filtered(logits, params.temperature, params.top_k, params.top_p,
                                params.repeat_penalty, dev_ids, dev_n, self.seq_state,
                                slots, out_ids)
