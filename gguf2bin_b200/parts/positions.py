"""Position encodings applied to queries and keys before the keys are cached.

``rope_neox``: half-split rotation, pairs (j, j + r/2) of the first r = rotary_dim
dimensions of each head, angle = pos * theta^(-2j/r) in float32
(src/l3_math.c:84-102 of AnonymoDGH/gguf2bin; r = head_dim there).  The frequencies
are a table handed to the fused norm+rotation kernel, so another encoding that only
changes the frequencies needs no kernel of its own.
``none``: nothing is applied.
"""
from __future__ import annotations

import torch

from ..config.specs import ConfigError, PartSpec
from .registry import register_position


_INV_FREQ: dict = {}


class RopeNeox:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, head_dim: int, device):
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or head_dim)
        if self.rotary_dim % 2 or not (0 < self.rotary_dim <= head_dim):
            raise ConfigError(f"rope_neox: rotary_dim {self.rotary_dim} must be even and at most "
                              f"head_dim {head_dim}")
        # one table per (theta, rotary_dim, device): layers with equal frequencies share the tensor,
        # and with it the step's (cos, sin) table
        key = (self.theta, self.rotary_dim, str(device))
        if key not in _INV_FREQ:
            j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
            _INV_FREQ[key] = (self.theta ** (-2.0 * j / self.rotary_dim)).to(torch.float32).to(device)
        self.inv_freq = _INV_FREQ[key]

    def fused_rotation(self):
        return self.inv_freq, self.rotary_dim

    def apply(self, q, k, ctx) -> None:          # never needed: the rotation is fused
        raise NotImplementedError


class NoPosition:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, head_dim: int, device):
        pass

    def fused_rotation(self):
        return None, 0                           # fused path with no rotation

    def apply(self, q, k, ctx) -> None:
        pass


register_position("rope_neox", RopeNeox)
register_position("none", NoPosition)
