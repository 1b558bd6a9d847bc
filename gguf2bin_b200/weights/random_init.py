"""Random-weights mode: writes a model folder (config.json + model.safetensors) from a
configuration and a seed.

Matrices are N(0, std) and scale vectors (norm weights) 1 + N(0, scale_std); the
reference's own synthetic model (src/l5_model.c:622-680) has all-zero matrices and
unit norms, which hides every fault, so it is not imitated.  Each tensor is drawn from
its own generator keyed by (seed, position of the tensor in the model's list), so a
tensor's values do not depend on the others.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch

from .loader import Expected
from .safetensors_io import write_safetensors


def random_tensor(e: Expected, seed: int, index: int, dtype: torch.dtype,
                  std: float, scale_std: float) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed((int(seed) * 1000003 + index * 7919 + 12345) % (2 ** 63))
    z = torch.randn(e.shape, generator=g, dtype=torch.float32)
    if e.init == "scale":
        z = 1.0 + scale_std * z
    elif e.init == "matrix":
        z = std * z
    else:
        raise ValueError(f"unknown init kind {e.init!r}")
    return z.to(dtype)


def write_random_model(folder, config: Mapping, seed: int, dtype: str = "bfloat16",
                       std: float = 0.02, scale_std: float = 0.1,
                       expected: Mapping[str, Expected] | None = None) -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``.  ``dtype`` is the
    storage type of every tensor ("bfloat16" or "float32").  ``expected`` defaults to the
    tensors of the model that ``config`` describes."""
    from ..engine.model import expected_tensors          # late: engine imports weights
    from ..config import model_spec_from_dict

    tdtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    if expected is None:
        expected = expected_tensors(model_spec_from_dict(config))
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    cfg = dict(config)
    cfg["torch_dtype"] = dtype
    (folder / "config.json").write_text(json.dumps(cfg, indent=1))
    items = []
    for i, (name, e) in enumerate(expected.items()):
        if e.optional:
            continue
        items.append((name, tuple(e.shape), tdtype,
                      (lambda e=e, i=i: random_tensor(e, seed, i, tdtype, std, scale_std))))
    write_safetensors(folder / "model.safetensors", items)
    return folder
