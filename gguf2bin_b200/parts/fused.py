"""Products that start from the residual stream: ``linear(norm(x))``.

The norm part runs first into scratch memory and the product follows (with the SiLU gate in
its epilogue when a kernel takes the case).  Folding an RMSNorm into the prologue of the
few-row product was tried and measured: every 16-row tile of the product repeats the norm of
all rows, and the norm as a kernel of its own (1.4 us at eight rows) is faster.
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
    h = ctx.workspace.buffer("fused.normed", (n, x32.shape[1]), ctx.dtype)
    norm.forward(x32, h, rows)
    if gate_block is None:
        kernels.linear(h, w, out)
    elif not kernels.gate_up_fused(h, w, out, gate_block):
        gu = ctx.workspace.buffer("fused.gate_up", (n, w.shape[0]), ctx.dtype)
        kernels.linear(h, w, gu)
        kernels.swiglu(gu, out, gate_block)
