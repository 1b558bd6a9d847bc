"""Feed-forwards.  ``swiglu``: down( silu(gate x) * (up x) ), no bias, dense
(src/l5_model.c:588-597, silu src/l3_math.c:57-62 of AnonymoDGH/gguf2bin).

The gate and up matrices are fused into one at bind time, rows alternating in blocks of
eight (eight gate rows, then the eight up rows of the same outputs), so one product
yields both and a kernel finds a gate and its up value sixteen columns apart at most.
A width that is no multiple of eight keeps the plain order (all gates, then all ups).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.specs import PartSpec
from ..weights.loader import Expected
from .fused import normed_linear
from .registry import register_feed_forward


class SwiGLU:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.inter = int(spec["intermediate_size"])
        self.hidden = int(hidden_size)
        self.block = 8 if self.inter % 8 == 0 else self.inter
        self.dtype = dtype
        self.names = dict(spec["names"])
        self.w_gate_up = self.w_down = None

    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n, inter = dict(spec["names"]), spec["intermediate_size"]
        return {n["gate"]: Expected((inter, hidden_size)), n["up"]: Expected((inter, hidden_size)),
                n["down"]: Expected((hidden_size, inter))}

    def bind(self, tensors: dict) -> None:
        g, u = tensors[self.names["gate"]], tensors[self.names["up"]]
        if g.dtype != u.dtype:
            g, u = g.to(torch.float32), u.to(torch.float32)
        b = self.block
        fused = torch.stack([g.view(self.inter // b, b, self.hidden),
                             u.view(self.inter // b, b, self.hidden)], dim=1)
        self.w_gate_up = fused.reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def weights(self):
        return (self.w_gate_up, self.w_down)

    def absorb_norm_weight(self, norm) -> bool:
        """As ``GQAAttention.absorb_norm_weight``, into the columns of the gate/up matrix."""
        if self.dtype != torch.bfloat16 or self.w_gate_up.dtype != torch.bfloat16 or self.block != 8 \
                or not hasattr(norm, "give_up_weight"):
            return False
        w = norm.give_up_weight()
        self.w_gate_up = (self.w_gate_up.float() * w.to(self.w_gate_up.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def notices(self) -> list:
        return (kernels.product_notices("feed-forward gate/up", self.w_gate_up, self.dtype)
                + kernels.product_notices("feed-forward down", self.w_down, self.dtype))

    def forward(self, h: torch.Tensor, ctx, residual32: torch.Tensor) -> None:
        T = h.shape[0]
        ws = ctx.workspace
        mid = ws.buffer("ffn.mid", (T, self.inter), self.dtype)
        if not kernels.gate_up_fused(h, self.w_gate_up, mid, self.block):
            gu = ws.buffer("ffn.gate_up", (T, 2 * self.inter), self.dtype)
            kernels.linear(h, self.w_gate_up, gu)
            kernels.swiglu(gu, mid, self.block)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)

    def forward_from_stream(self, x32: torch.Tensor, norm, ctx, residual32: torch.Tensor) -> None:
        """The same with the block's norm folded into the gate/up product."""
        mid = ctx.workspace.buffer("ffn.mid", (x32.shape[0], self.inter), self.dtype)
        normed_linear(x32, norm, self.w_gate_up, mid, ctx, gate_block=self.block)
        kernels.linear(mid, self.w_down, residual32, accumulate=True)


register_feed_forward("swiglu", SwiGLU)
