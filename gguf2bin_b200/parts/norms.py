"""Norms.  ``rmsnorm``: o_j = (w_j * x_j) / sqrt(mean(x^2) + eps), statistics in float32,
the weight a plain multiplier (src/l3_math.c:21-51 of AnonymoDGH/gguf2bin)."""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import PartSpec
from ..weights.loader import Expected
from .registry import register_norm


class RMSNorm:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, width: int, dtype: torch.dtype, device):
        self.eps = float(spec["eps"])
        self.width = int(width)
        self.weight = None

    @classmethod
    def expected(cls, spec: PartSpec, width: int, name: str) -> dict:
        return {name: Expected((int(width),), init="scale")}

    def bind(self, weight: torch.Tensor) -> None:
        self.weight = weight.to(torch.float32).contiguous()      # exact widening

    def weights(self):
        return (self.weight,) if self.weight is not None else ()

    # ---- the weight moved into the matrix that follows ----------------------------------
    def give_up_weight(self) -> torch.Tensor:
        """Hands the per-channel weight to a part that multiplies it into the columns of its
        first matrix (W' = W . diag(w), so that W' . x/rms(x) = W . (w * x/rms(x))); from
        then on this norm only divides by the root mean square."""
        w, self.weight = self.weight, None
        return w

    def plain_rms_eps(self):
        """eps when this norm is x / sqrt(mean(x^2) + eps) and nothing else (its weight was
        given up), which is what the products that normalise their own input take; else None."""
        return self.eps if self.weight is None else None

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows=None) -> None:
        kernels.rmsnorm(x32, self.weight, self.eps, out, rows)


register_norm("rmsnorm", RMSNorm)
