"""Binding checkpoint tensors to the names a model expects.

The model (its parts) says which tensors it needs: name, shape and kind.  The loader
finds them by exact name, checks every shape, and reports everything that is wrong in
ONE error: missing tensors, unexpected tensors and wrong shapes together.  Nothing is
defaulted: the reference fills a missing norm weight with zeros
(src/l5_model.c:438-439) and discovers a missing matrix only inside the forward pass
(src/l5_model.c:454-459); here both are load errors.

Precision policy: with compute dtype bfloat16, tensors stored as BF16 stay bfloat16,
F16 becomes bfloat16, and a tensor stored in 32-bit floating point stays 32-bit;
integer tables become int32.  With compute dtype float32 every floating tensor is
widened to float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Mapping

import torch

from .safetensors_io import SafetensorsFile, WeightsError, open_model_files


@dataclass(frozen=True)
class Expected:
    """A tensor the model needs.  ``init`` tells the random-weights writer how to fill
    it: "matrix" (N(0, std)) or "scale" (1 + N(0, scale_std)).  ``optional`` tensors may
    be absent (an lm_head matrix beside tied embeddings)."""
    shape: tuple
    init: str = "matrix"
    optional: bool = False


def runtime_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names_and_shapes(expected: Mapping[str, Expected],
                           found: Mapping[str, tuple]) -> None:
    """Raises one ``WeightsError`` listing all missing, unexpected and misshapen tensors."""
    missing = [n for n, e in expected.items() if n not in found and not e.optional]
    unexpected = [n for n in found if n not in expected]
    wrong = [(n, tuple(found[n]), tuple(e.shape)) for n, e in expected.items()
             if n in found and tuple(found[n]) != tuple(e.shape)]
    if not (missing or unexpected or wrong):
        return
    lines = ["weights do not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}):")
        lines += [f"    {n}  expected shape {list(expected[n].shape)}" for n in missing]
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}):")
        lines += [f"    {n}  shape {list(found[n])}" for n in unexpected]
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}):")
        lines += [f"    {n}  found {list(f)}, expected {list(e)}" for n, f, e in wrong]
    raise WeightsError("\n".join(lines))


def load_weights(folder, expected: Mapping[str, Expected], compute_dtype: torch.dtype,
                 device) -> dict[str, torch.Tensor]:
    """name -> tensor on ``device`` for every expected tensor that the folder has."""
    files = open_model_files(folder)
    try:
        where: dict[str, SafetensorsFile] = {}
        dup = []
        for f in files:
            for name in f.entries:
                if name in where:
                    dup.append(name)
                where[name] = f
        if dup:
            raise WeightsError("tensors present in more than one shard: " + ", ".join(sorted(dup)))
        check_names_and_shapes(expected, {n: f.entries[n].shape for n, f in where.items()})
        out = {}
        for name in expected:
            if name not in where:
                continue
            cpu = where[name].tensor(name)
            out[name] = cpu.to(device=device, dtype=runtime_dtype(cpu.dtype, compute_dtype),
                               copy=True)
            del cpu
        return out
    finally:
        for f in files:
            f.close()
