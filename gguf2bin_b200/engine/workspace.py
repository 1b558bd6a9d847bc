"""Scratch memory of a step: named device buffers that grow to the largest request and
are then reused, so that steady-state steps allocate nothing (which is also what lets a
step be captured in a CUDA graph)."""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self._buffers: dict[str, torch.Tensor] = {}
        self._views: dict = {}         # (name, shape, dtype) -> view of the buffer as it is now
        self.generation = 0            # bumps whenever a buffer moves (captured graphs go stale)

    def buffer(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        key = (name, tuple(shape), dtype)
        view = self._views.get(key)
        if view is not None:
            return view
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * dtype.itemsize
        raw = self._buffers.get(name)
        if raw is None or raw.numel() < nbytes:
            # room to spare, so a slowly growing batch does not reallocate every step
            cap = max(nbytes, 256) if raw is None else max(nbytes, 2 * raw.numel())
            raw = torch.empty(cap, dtype=torch.uint8, device=self.device)
            self._buffers[name] = raw
            self.generation += 1
            self._views = {k: v for k, v in self._views.items() if k[0] != name}
        if len(self._views) > 4096:    # many distinct step sizes: start over rather than grow
            self._views.clear()
        view = raw[:nbytes].view(dtype).view(*shape)
        self._views[key] = view
        return view

    def bytes(self) -> int:
        return sum(b.numel() for b in self._buffers.values())
