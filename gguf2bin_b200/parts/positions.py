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
        self.head_dim = int(head_dim)
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

    def apply(self, q, k, ctx) -> None:
        """Rotates q [T, heads*head_dim] and k in place.  The library's own mixer never comes
        here (it hands ``fused_rotation()`` to its fused kernel); a mixer that runs its
        position part as a step of its own does.  The rotation is that same kernel's, asked
        for nothing but the rotation."""
        from .. import kernels
        rope = ctx.rope_table(self.inv_freq)
        for i, a in enumerate((q, k)):
            if a is None or a.numel() == 0:
                continue
            out = ctx.workspace.buffer(f"rope.apply.{i}", tuple(a.shape), a.dtype)
            kernels.qknorm_rope_cache(a, a.shape[1] // self.head_dim, 0, self.head_dim, None, None,
                                      0.0, rope, self.rotary_dim, ctx.tok_pos, ctx.tok_seq, None,
                                      None, ctx.page_size, out)
            a.copy_(out)


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
