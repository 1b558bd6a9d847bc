"""Products that start from the residual stream: ``linear(norm(x))``.

The norm part runs first into scratch memory and the product follows (with the SiLU gate in
its epilogue when a kernel takes the case).  One case needs no norm kernel: when the norm has
given its per-channel weight to the matrix (``norm.plain_rms_eps()``), what is left of it is
one factor per row, and the few-row product applies that factor to its accumulators while it
sums the squares of the rows it stages anyway (``kernels.normed_product``).  Normalising the
rows in the product's prologue instead was tried and was slower than a norm kernel: every
16-row tile repeated the normalisation and its stores, not just the sum.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


def normed_linear(x32: torch.Tensor, norm, w: torch.Tensor, out: torch.Tensor, ctx,
                  rows: Optional[torch.Tensor] = None, gate_block: Optional[int] = None) -> None:
    """out = norm(x32[rows]) @ w.T, or, with ``gate_block``, out = silu(gate) * up of a fused
    gate/up matrix whose rows alternate ``gate_block`` gates and ups."""
    n = out.shape[0]
    eps = getattr(norm, "plain_rms_eps", lambda: None)()
    if eps is not None and rows is None and kernels.normed_product(x32, eps, w, out, gate_block):
        return
    h = ctx.workspace.buffer("fused.normed", (n, x32.shape[1]), ctx.dtype)
    norm.forward(x32, h, rows)
    if gate_block is None:
        kernels.linear(h, w, out)
    elif not kernels.gate_up_fused(h, w, out, gate_block):
        gu = ctx.workspace.buffer("fused.gate_up", (n, w.shape[0]), ctx.dtype)
        kernels.linear(h, w, gu)
        kernels.swiglu(gu, out, gate_block)
