"""Sequence mixers.  ``gqa_attention``: causal grouped-query attention over the cache.

Order of operations (src/l5_model.c:497-583 of AnonymoDGH/gguf2bin): q, k, v projections
without bias; per-head RMSNorm of q and k (if the spec has ``qk_norm``); position
encoding of q and k; k (normed, rotated) and v (raw) written to the cache; scores
(q . k) * scale over the keys up to the token's own position (optionally only the last
``window`` of them); softmax; weighted values; output projection added to the residual.

With ``shared_kv`` the mixer has no k and v projections and writes nothing: it attends
over the keys and values that another layer stored (the schedule entry's ``cache_of``
names that layer, whose kv heads and head size it must share).
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..cache.storage import KVNeed, KVView
from ..config.specs import ConfigError, PartSpec
from ..weights.loader import Expected
from .fused import normed_linear
from .registry import norm_class, position_class, register_mixer


class GQAAttention:
    def __init__(self, spec: PartSpec, hidden_size: int, dtype: torch.dtype, device):
        self.nh = int(spec["n_heads"])
        self.nkv = int(spec["n_kv_heads"])
        self.hd = int(spec["head_dim"])
        self.hidden = int(hidden_size)
        self.window = int(spec.get("window") or 0)
        self.shared_kv = bool(spec.get("shared_kv") or False)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv:
            raise ConfigError(f"gqa_attention: {self.nh} heads are not a multiple of "
                              f"{self.nkv} kv heads")
        if self.hd <= 0 or self.hd > 512:
            raise ConfigError(f"gqa_attention: head_dim {self.hd} outside 1..512")
        self.dtype, self.device = dtype, device
        self.names = dict(spec["names"])
        qk = spec.get("qk_norm")
        self.qk_eps = 0.0
        self.has_qk_norm = qk is not None
        if qk is not None:
            if qk.kind != "rmsnorm":
                raise ConfigError(f"gqa_attention: qk_norm of kind {qk.kind!r} is not supported")
            norm_class(qk)                            # must be registered
            self.qk_eps = float(qk["eps"])
        pos = spec.get("position") or PartSpec.make("none")
        self.position = position_class(pos)(pos, self.hd, device)
        self.w_qkv = self.w_o = self.q_norm_w = self.k_norm_w = None

    # ---- weights -------------------------------------------------------------
    @classmethod
    def expected(cls, spec: PartSpec, hidden_size: int) -> dict:
        n = dict(spec["names"])
        nq, nk = spec["n_heads"] * spec["head_dim"], spec["n_kv_heads"] * spec["head_dim"]
        shared = bool(spec.get("shared_kv") or False)
        out = {n["q"]: Expected((nq, hidden_size)), n["o"]: Expected((hidden_size, nq))}
        if not shared:
            out[n["k"]] = Expected((nk, hidden_size))
            out[n["v"]] = Expected((nk, hidden_size))
        if spec.get("qk_norm") is not None:
            out[n["q_norm"]] = Expected((spec["head_dim"],), init="scale")
            if not shared:
                out[n["k_norm"]] = Expected((spec["head_dim"],), init="scale")
        return out

    def bind(self, tensors: dict) -> None:
        n = self.names
        parts = [tensors[n["q"]]] if self.shared_kv else \
            [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_qkv = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.has_qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            if not self.shared_kv:
                self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()

    def weights(self):
        return [t for t in (self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w) if t is not None]

    def absorb_norm_weight(self, norm) -> bool:
        """Takes the weight of the norm in front of this mixer into the columns of the q/k/v
        matrix, when that is what makes the decode step shorter: bfloat16 compute and a
        bfloat16 matrix (the product then normalises its own rows, see ``parts/fused.py``).
        The matrix is rounded to bfloat16 once more; the 32-bit path keeps the formula's order."""
        if self.dtype != torch.bfloat16 or self.w_qkv.dtype != torch.bfloat16 or not hasattr(norm, "give_up_weight"):
            return False
        w = norm.give_up_weight()
        self.w_qkv = (self.w_qkv.float() * w.to(self.w_qkv.device)[None, :]).to(torch.bfloat16).contiguous()
        return True

    def notices(self) -> list:
        from ..cache.storage import PAGE_SIZE
        return (kernels.product_notices("attention q/k/v", self.w_qkv, self.dtype)
                + kernels.product_notices("attention output", self.w_o, self.dtype)
                + kernels.attention_notices("attention", self.hd, PAGE_SIZE, self.dtype))

    @property
    def graph_safe(self) -> bool:
        """Its own step only launches kernels; whether the whole of it may be replayed from a
        CUDA graph is then up to its position part."""
        return bool(getattr(self.position, "graph_safe", False))

    # ---- cache ---------------------------------------------------------------
    def cache_need(self):
        return None if self.shared_kv else KVNeed(self.nkv, self.hd, self.window)

    # ---- step ----------------------------------------------------------------
    def forward(self, h: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor) -> None:
        T = h.shape[0]
        nk = (0 if self.shared_kv else self.nkv) * self.hd
        qkv = ctx.workspace.buffer("attn.qkv", (T, self.nh * self.hd + 2 * nk), self.dtype)
        kernels.linear(h, self.w_qkv, qkv)
        self._attend(qkv, ctx, view, residual32)

    def forward_from_stream(self, x32: torch.Tensor, norm, ctx, view: KVView,
                            residual32: torch.Tensor) -> None:
        """The same with the block's norm folded into the q/k/v product."""
        T = x32.shape[0]
        nk = (0 if self.shared_kv else self.nkv) * self.hd
        qkv = ctx.workspace.buffer("attn.qkv", (T, self.nh * self.hd + 2 * nk), self.dtype)
        normed_linear(x32, norm, self.w_qkv, qkv, ctx)
        self._attend(qkv, ctx, view, residual32)

    def _attend(self, qkv: torch.Tensor, ctx, view: KVView, residual32: torch.Tensor) -> None:
        T = qkv.shape[0]
        nq = self.nh * self.hd
        nkv_own = 0 if self.shared_kv else self.nkv        # kv heads this layer projects
        nk = nkv_own * self.hd
        ws = ctx.workspace
        q = ws.buffer("attn.q", (T, nq), self.dtype)
        fused = self.position.fused_rotation()
        if fused is not None:
            inv_freq, rot = fused
            rope = ctx.rope_table(inv_freq) if inv_freq is not None else None
            kernels.qknorm_rope_cache(qkv, self.nh, nkv_own, self.hd, self.q_norm_w,
                                      self.k_norm_w, self.qk_eps, rope, rot, ctx.tok_pos,
                                      ctx.tok_seq, ctx.page_table, view.pages, view.page_size, q)
        else:
            k = ws.buffer("attn.k", (T, nk), self.dtype)
            v = ws.buffer("attn.v", (T, nk), self.dtype)
            kernels.qknorm_rope_cache(qkv, self.nh, nkv_own, self.hd, self.q_norm_w,
                                      self.k_norm_w, self.qk_eps, None, 0, ctx.tok_pos,
                                      ctx.tok_seq, None, None, view.page_size, q, k, v)
            self.position.apply(q, k, ctx)
            if nkv_own:
                kernels.cache_write(k, v, self.nkv, self.hd, ctx.tok_pos, ctx.tok_seq,
                                    ctx.page_table, view.pages, view.page_size)
        o = ws.buffer("attn.o", (T, nq), self.dtype)
        kernels.attention(q, o, view.pages, ctx, self.nh, self.nkv, self.hd, view.page_size,
                          self.window, self.scale)
        kernels.linear(o, self.w_o, residual32, accumulate=True)


register_mixer("gqa_attention", GQAAttention)
