"""A model: parts built from a ``ModelSpec``, weights bound by name, and the forward
pass of one step over the residual stream.

The forward pass is the reference's (src/l5_model.c:488-605 of AnonymoDGH/gguf2bin):
embedding rows, the scheduled layers, final norm and lm_head — the last two only on the
rows whose logits are wanted.
"""
from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch

from .. import kernels
from ..cache.storage import Cache
from ..config import ModelSpec, model_spec_from_folder
from ..config.specs import ConfigError
from ..csrc.build import _log
from ..parts import block_class, embedding_class, head_class, norm_class
from ..parts.base import StepContext
from ..weights.loader import load_weights

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ConfigError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


def expected_tensors(spec: ModelSpec) -> dict:
    """Every tensor the model needs, by checkpoint name."""
    out = dict(embedding_class(spec.embedding).expected(spec.embedding, spec.vocab_size,
                                                        spec.hidden_size))
    out.update(norm_class(spec.final_norm).expected(spec.final_norm, spec.hidden_size,
                                                    spec.final_norm["name"]))
    out.update(head_class(spec.head).expected(spec.head, spec.vocab_size, spec.hidden_size))
    for layer in spec.layers:
        for name, e in block_class(layer.block).expected(layer, spec.hidden_size).items():
            out[layer.prefix + name] = e
    return out


class Model:
    def __init__(self, spec: ModelSpec, dtype="bfloat16", device="cuda:0"):
        spec.validate()
        self.spec = spec
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise kernels.KernelError("the engine runs on a CUDA device only (no CPU path)")
        if not torch.cuda.is_available():
            raise kernels.KernelError("no CUDA device is available (no NVIDIA driver or no GPU); "
                                      "the engine has no CPU path")
        self.hidden, self.vocab = spec.hidden_size, spec.vocab_size
        self.blocks = [block_class(l.block)(l, spec.hidden_size, self.dtype, self.device)
                       for l in spec.layers]
        self.final_norm = norm_class(spec.final_norm)(spec.final_norm, spec.hidden_size,
                                                      self.dtype, self.device)
        self.embedding = embedding_class(spec.embedding)(spec.embedding, spec.vocab_size,
                                                         spec.hidden_size, self.dtype, self.device)
        self.head = head_class(spec.head)(spec.head, spec.vocab_size, spec.hidden_size, self.dtype,
                                          self.device)
        self.n_params = 0

    # ---- construction ---------------------------------------------------------
    @classmethod
    def from_folder(cls, folder, dtype="bfloat16", device="cuda:0") -> "Model":
        """The model class comes from config.json's architecture through the registry."""
        spec = model_spec_from_folder(folder)
        model = cls(spec, dtype, device)
        tensors = load_weights(Path(folder), expected_tensors(spec), model.dtype, model.device)
        model.bind(tensors)
        return model

    @classmethod
    def random(cls, config, seed: int, dtype="bfloat16", device="cuda:0", storage=None,
               std: float = 0.02, scale_std: float = 0.1) -> "Model":
        """A model with random weights made in device memory, never touching the disk:
        ``config`` is a config.json dictionary (read through the registry) or a ``ModelSpec``.
        The weights are those of ``write_random_model(folder, config, seed, storage)`` loaded
        with ``dtype``, bit for bit (``storage`` defaults to the compute dtype).  The
        reference makes its synthetic model in-process as well (src/l5_model.c:634-680)."""
        from ..config import model_spec_from_dict
        from ..weights.random_init import random_tensors_on_device
        spec = config if isinstance(config, ModelSpec) else model_spec_from_dict(config)
        model = cls(spec, dtype, device)
        stored = parse_dtype(storage) if storage is not None else model.dtype
        with torch.cuda.device(model.device):
            tensors = random_tensors_on_device(expected_tensors(spec), seed, stored, model.dtype,
                                               model.device, std, scale_std)
            model.bind(tensors)
        return model

    def bind(self, tensors: dict) -> None:
        spec = self.spec
        self.n_params = sum(t.numel() for t in tensors.values())
        self.embedding.bind(tensors)
        self.head.bind(tensors, self.embedding)      # a tied head takes the embedding's table
        self.final_norm.bind(tensors[spec.final_norm["name"]])
        for layer, block in zip(spec.layers, self.blocks):
            n = len(layer.prefix)
            block.bind({k[n:]: v for k, v in tensors.items() if k.startswith(layer.prefix)})
        for line in self.notices():
            _log("note: " + line)

    def notices(self) -> list:
        """What the parts say about kernels they will not get (a head size without a tensor-core
        attention kernel, a matrix kept in 32-bit under bfloat16 compute): each distinct line
        once, with the layers it holds for."""
        where: dict = {}
        for i, b in enumerate(self.blocks):
            for line in getattr(b, "notices", list)():
                where.setdefault(line, []).append(str(i))
        out = [f"layers {','.join(ls) if len(ls) <= 4 else ls[0] + '..' + ls[-1]}: {line}"
               for line, ls in where.items()]
        for part in (self.embedding, self.head):
            out += getattr(part, "notices", list)()
        return out

    # ---- cache ----------------------------------------------------------------
    def cache_needs(self) -> list:
        """The need of each schedule position: what its layer asks for, or None when the
        position borrows another position's storage or its layer stores nothing."""
        return [self.blocks[e.layer].cache_need() if e.cache_of is None else None
                for e in self.spec.schedule]

    def new_cache(self, max_tokens: int, max_seqs: Optional[int] = None) -> Cache:
        return Cache(self.cache_needs(), max_tokens, self.dtype, self.device, max_seqs)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._all_weights():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _all_weights(self):
        """Every tensor a part says it holds (a part without ``weights()`` reports none)."""
        for part in (self.embedding, self.head, self.final_norm, *self.blocks):
            for t in getattr(part, "weights", tuple)():
                if t is not None:
                    yield t

    def describe(self) -> str:
        s = self.spec
        return (f"{s.architecture}: {len(s.layers)} layers, width {s.hidden_size}, vocab "
                f"{s.vocab_size}, {self.n_params / 1e6:.1f} M parameters, "
                f"{self.weight_bytes() / 2**20:.1f} MiB, compute {self.dtype}")

    @property
    def graph_safe(self) -> bool:
        """True when every part of every block declares that its step may be replayed from a
        CUDA graph; one part that does not (a part registered from outside, say) makes all steps
        of this model run plainly."""
        return all(getattr(part, "graph_safe", False)
                   for part in (self.embedding, self.final_norm, self.head, *self.blocks))

    # ---- one step ---------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: Cache, want_rows: Optional[torch.Tensor],
                n_want: int, logits_out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the step's tokens through the scheduled layers.  ``want_rows`` (int32
        [n_want]) are the token indices whose logits are returned as float32 [n_want, V];
        with ``n_want == 0`` only the cache is updated."""
        ws = ctx.workspace
        ctx.step_cache.clear()                     # per-step tables are rebuilt from this step's tokens
        x = ws.buffer("stream", (ctx.n_tokens, self.hidden), torch.float32)
        self.embedding.forward(ctx.tok_ids[:ctx.n_tokens], x, ctx)
        for position, entry in enumerate(self.spec.schedule):
            self.blocks[entry.layer].forward(x, ctx, cache.view(self.spec.cache_owner(position)))
        if n_want == 0:
            return None
        logits = logits_out if logits_out is not None else \
            ws.buffer("head.logits", (n_want, self.vocab), torch.float32)
        h = ws.buffer("head.normed", (n_want, self.hidden), self.dtype)
        self.final_norm.forward(x, h, want_rows)
        self.head.forward(h, logits, ctx)
        return logits
