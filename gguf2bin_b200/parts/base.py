"""What every part gets and must offer.

Common rules
* A part is built from its ``PartSpec`` plus the sizes of its surroundings (the model
  width, the compute dtype, the device).  It never sees the model or the architecture.
* ``expected(spec, ...)`` (a classmethod) lists the tensors the part needs as
  ``{checkpoint name relative to the layer prefix: Expected}``; ``bind(tensors)`` receives
  them under the same names once loaded and may fuse or re-lay them.
* ``forward`` launches kernels on the current stream, allocates only through
  ``ctx.workspace`` and returns nothing that lives longer than the step.

Norm          forward(x32 [T,H] float32, out [T,H] compute dtype, rows=None)
Position      fused_rotation() -> (inv_freq float32 [r/2], rotary_dim) or None;
              apply(q [T,nh*hd], k [T,nkv*hd], ctx) in place when it cannot be fused
Mixer         cache_need() -> KVNeed | StateNeed | None;
              forward(h [T,H], ctx, cache_view, residual32 [T,H]): ADDS its output
Feed-forward  forward(h [T,H], ctx, residual32 [T,H]): ADDS its output
Block         forward(x32 [T,H], ctx, cache_view): one whole layer on the residual stream
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch


ATTN_TILE_ROWS = 64          # query rows per work item of the prompt attention kernel (mma.sync)
ATTN_WIDE_TILE_ROWS = 128    # ... of the tcgen05 prompt attention kernel


@dataclass
class StepContext:
    """One step's batch as the kernels see it.  All index tensors are int32 on the device.

    tok_ids [T]      token ids, sequences one after another
    tok_pos [T]      absolute position of each token in its sequence
    tok_seq [T]      index (0..B-1) of each token's sequence in this step
    page_table [B,P] pages of each sequence, in position order
    Host-side copies (lists) describe the same batch for parts that plan launches.
    """
    n_tokens: int
    n_seqs: int
    tok_ids: torch.Tensor
    tok_pos: torch.Tensor
    tok_seq: torch.Tensor
    page_table: torch.Tensor
    page_size: int
    workspace: "object"
    dtype: torch.dtype
    q_lens: list = field(default_factory=list)       # tokens of each sequence in this step
    past_lens: list = field(default_factory=list)    # tokens each sequence held before it
    slots: list = field(default_factory=list)        # slot of each sequence
    max_kv_len: int = 0                              # longest sequence after this step (a replayed decode step: its upper bound)
    kv_len_hint: int = 0                             # where max_kv_len is an upper bound: the longest sequence as of now (0: unknown)
    seq_meta: Optional[torch.Tensor] = None          # [B,4] int32: q_start, q_len, past, slot
    attn_tiles: Optional[torch.Tensor] = None        # [n,4] int32: sequence, first token, rows, position
    n_attn_tiles: int = 0                            # of row 0; tiles of ATTN_TILE_ROWS query rows
    attn_tiles_wide: Optional[torch.Tensor] = None   # the same with ATTN_WIDE_TILE_ROWS rows (tcgen05 kernel)
    n_attn_tiles_wide: int = 0
    step_cache: dict = field(default_factory=dict)   # tensors derived once per step (cleared by the model)

    def rope_table(self, inv_freq: torch.Tensor) -> torch.Tensor:
        """(cos, sin) of every token's position times ``inv_freq``, computed once per step and
        shared by all layers that rotate with these frequencies; float32 [T, half, 2]."""
        key = ("rope", inv_freq.data_ptr())
        table = self.step_cache.get(key)
        if table is None:
            from .. import kernels
            table = self.workspace.buffer(f"rope.table.{len(self.step_cache)}",
                                          (self.n_tokens, inv_freq.shape[0], 2), torch.float32)
            kernels.rope_table(self.tok_pos[:self.n_tokens], inv_freq, table)
            self.step_cache[key] = table
        return table

    @property
    def all_single(self) -> bool:
        return self.n_tokens == self.n_seqs
