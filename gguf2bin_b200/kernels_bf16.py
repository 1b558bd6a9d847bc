"""Bindings of the bfloat16 tensor-core kernels.  Each function returns True when it ran,
False when it does not take the case (the caller then uses the 32-bit kernel)."""
from __future__ import annotations

import torch


def linear_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> bool:
    return False


def gate_up_bf16(h: torch.Tensor, w_gate_up: torch.Tensor, mid: torch.Tensor, block: int) -> bool:
    return False


def attention_bf16(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
                   scale) -> bool:
    return False
