"""The two ends of a model: token ids into the residual stream, and the residual stream
into logits.

``token_embedding``: row ``id`` of the table, widened to float32
(src/l5_model.c:488-492 of AnonymoDGH/gguf2bin).
``lm_head``: logits = h . W^T in float32, W a matrix of its own or, when ``tied``, the
embedding's table (src/l5_model.c:600-605: without an output tensor the reference
multiplies by the token-embedding matrix).

Another architecture's ends (a scaled embedding, a logit scale or cap, a bias) are other
kinds of these two families; the model only walks parts.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .registry import register_embedding, register_head


class TokenEmbedding:
    graph_safe = True          # its step only launches kernels: may be replayed from a CUDA graph

    def __init__(self, spec: PartSpec, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.name = spec["name"]
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.table: Optional[torch.Tensor] = None      # [vocab, hidden]; a tied head multiplies by it

    @classmethod
    def expected(cls, spec: PartSpec, vocab_size: int, hidden_size: int) -> dict:
        return {spec["name"]: Expected((int(vocab_size), int(hidden_size)))}

    def bind(self, tensors: dict) -> None:
        self.table = tensors[self.name].contiguous()

    def weights(self):
        return (self.table,)

    def forward(self, tok_ids: torch.Tensor, out32: torch.Tensor, ctx) -> None:
        """out32[t] = table[tok_ids[t]] as float32; out32 is [T, hidden]."""
        kernels.embed_rows(self.table, tok_ids, out32)


class LMHead:
    graph_safe = True

    def __init__(self, spec: PartSpec, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.name = spec["name"]
        self.tied = bool(spec.get("tied") or False)
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.dtype = dtype
        self.matrix: Optional[torch.Tensor] = None

    @classmethod
    def expected(cls, spec: PartSpec, vocab_size: int, hidden_size: int) -> dict:
        # beside tied embeddings a checkpoint may or may not carry the (equal) matrix
        return {spec["name"]: Expected((int(vocab_size), int(hidden_size)),
                                       optional=bool(spec.get("tied") or False))}

    def bind(self, tensors: dict, embedding) -> None:
        if self.tied:
            table = getattr(embedding, "table", None)
            if table is None or tuple(table.shape) != (self.vocab, self.hidden):
                raise ConfigError("lm_head: tied, but the embedding part offers no table of "
                                  f"[{self.vocab}, {self.hidden}]")
            self.matrix = table
        else:
            self.matrix = tensors[self.name].contiguous()

    def weights(self):
        return (self.matrix,)

    def notices(self) -> list:
        return kernels.product_notices("lm_head", self.matrix, self.dtype)

    def forward(self, h: torch.Tensor, logits32: torch.Tensor, ctx) -> None:
        """logits32 [n, vocab] float32 = h [n, hidden] . matrix^T."""
        kernels.linear(h, self.matrix, logits32)


register_embedding("token_embedding", TokenEmbedding)
register_head("lm_head", LMHead)
