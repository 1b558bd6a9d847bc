"""Block arrangements.  ``prenorm``: x += mixer(norm(x)); x += feed_forward(norm(x)), the
residual stream kept in float32 (src/l5_model.c:494-597 of AnonymoDGH/gguf2bin)."""
from __future__ import annotations

import torch

from ..config.specs import LayerSpec
from .registry import (feed_forward_class, mixer_class, norm_class, register_block)


class PreNormBlock:
    def __init__(self, layer: LayerSpec, hidden_size: int, dtype: torch.dtype, device):
        self.names = dict(layer.block["names"])
        self.hidden, self.dtype = int(hidden_size), dtype
        ffn_norm = layer.ffn_norm or layer.norm
        self.mixer_norm = norm_class(layer.norm)(layer.norm, hidden_size, dtype, device)
        self.ffn_norm = norm_class(ffn_norm)(ffn_norm, hidden_size, dtype, device)
        self.mixer = mixer_class(layer.mixer)(layer.mixer, hidden_size, dtype, device)
        self.feed_forward = feed_forward_class(layer.feed_forward)(layer.feed_forward, hidden_size,
                                                                   dtype, device)

    @classmethod
    def expected(cls, layer: LayerSpec, hidden_size: int) -> dict:
        names = dict(layer.block["names"])
        ffn_norm = layer.ffn_norm or layer.norm
        out = {}
        out.update(norm_class(layer.norm).expected(layer.norm, hidden_size, names["mixer_norm"]))
        out.update(norm_class(ffn_norm).expected(ffn_norm, hidden_size, names["ffn_norm"]))
        out.update(mixer_class(layer.mixer).expected(layer.mixer, hidden_size))
        out.update(feed_forward_class(layer.feed_forward).expected(layer.feed_forward, hidden_size))
        return out

    def bind(self, tensors: dict) -> None:
        self.mixer_norm.bind(tensors[self.names["mixer_norm"]])
        self.ffn_norm.bind(tensors[self.names["ffn_norm"]])
        self.mixer.bind(tensors)
        self.feed_forward.bind(tensors)
        # a part that starts from the stream (``forward_from_stream``) may take the weight of
        # the norm in front of it into its first matrix; the norm is then a plain division
        for part, norm in ((self.mixer, self.mixer_norm), (self.feed_forward, self.ffn_norm)):
            if hasattr(part, "forward_from_stream") and hasattr(part, "absorb_norm_weight"):
                part.absorb_norm_weight(norm)

    def cache_need(self):
        return self.mixer.cache_need()

    def parts(self) -> tuple:
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)

    def weights(self):
        """Every tensor the block's parts hold (a part without ``weights()`` reports none)."""
        for part in self.parts():
            yield from getattr(part, "weights", tuple)()

    def notices(self) -> list:
        return [line for part in self.parts() for line in getattr(part, "notices", list)()]

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this block may be captured in a CUDA graph and replayed: every part
        must say so itself (``graph_safe = True``: its step does nothing but launch kernels on
        the current stream, takes its scratch memory from the step's workspace, and neither reads
        results on the host nor keeps host-side state from step to step)."""
        return all(getattr(part, "graph_safe", False) for part in self.parts())

    def forward(self, x32: torch.Tensor, ctx, cache_view) -> None:
        # a part that offers ``forward_from_stream`` takes the stream and the norm and may
        # fold the norm into its first product; any other part gets normed activations
        T = x32.shape[0]
        if hasattr(self.mixer, "forward_from_stream"):
            self.mixer.forward_from_stream(x32, self.mixer_norm, ctx, cache_view, x32)
        else:
            h = ctx.workspace.buffer("block.normed", (T, self.hidden), self.dtype)
            self.mixer_norm.forward(x32, h)
            self.mixer.forward(h, ctx, cache_view, x32)
        if hasattr(self.feed_forward, "forward_from_stream"):
            self.feed_forward.forward_from_stream(x32, self.ffn_norm, ctx, x32)
        else:
            h = ctx.workspace.buffer("block.normed", (T, self.hidden), self.dtype)
            self.ffn_norm.forward(x32, h)
            self.feed_forward.forward(h, ctx, x32)


register_block("prenorm", PreNormBlock)
