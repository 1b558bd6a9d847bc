"""Products that start from the residual stream: ``linear(norm(x))``.

The norm is computed inside the product's prologue when a kernel takes the case (RMSNorm,
bfloat16 weights, few rows: the decode step), which saves a kernel launch and a round trip
of the normed activations through memory; otherwise the norm part runs first into scratch
memory and the plain product follows.  Either way the result is the same function of the
same inputs.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels


FUSE_MAX_ROWS = 16
FUSE_MAX_OUTPUTS = 4096


def _rms_params(norm):
    """(weight, eps) when ``norm`` is an RMSNorm whose formula the fused kernels implement."""
    from .norms import RMSNorm
    if type(norm) is RMSNorm and norm.weight is not None:
        return norm.weight, norm.eps
    return None


def normed_linear(x32: torch.Tensor, norm, w: torch.Tensor, out: torch.Tensor, ctx,
                  rows: Optional[torch.Tensor] = None, gate_block: Optional[int] = None) -> None:
    """out = norm(x32[rows]) @ w.T, or, with ``gate_block``, out = silu(gate) * up of a fused
    gate/up matrix whose rows alternate ``gate_block`` gates and ups."""
    from .. import kernels_bf16
    rms = _rms_params(norm)
    # every 16-row tile of the product repeats the norm of all rows, so folding pays only
    # for few rows and few tiles; beyond that the norm runs once, as a kernel of its own
    few = out.shape[0] <= FUSE_MAX_ROWS and w.shape[0] <= FUSE_MAX_OUTPUTS
    if few and rms is not None and w.dtype == torch.bfloat16 and ctx.dtype == torch.bfloat16:
        if gate_block is None:
            if kernels_bf16.linear_normed_bf16(x32, rms[0], rms[1], rows, w, out):
                return
        elif gate_block == 8 and w.shape[0] % 16 == 0 and out.dtype == torch.bfloat16:
            if kernels_bf16.linear_normed_bf16(x32, rms[0], rms[1], rows, w, out,
                                               kernels_bf16.EPI_SWIGLU_BF16):
                return
    n = out.shape[0]
    h = ctx.workspace.buffer("fused.normed", (n, x32.shape[1]), ctx.dtype)
    norm.forward(x32, h, rows)
    if gate_block is None:
        kernels.linear(h, w, out)
    elif not kernels.gate_up_fused(h, w, out, gate_block):
        gu = ctx.workspace.buffer("fused.gate_up", (n, w.shape[0]), ctx.dtype)
        kernels.linear(h, w, gu)
        kernels.swiglu(gu, out, gate_block)
