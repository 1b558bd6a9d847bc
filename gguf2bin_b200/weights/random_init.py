"""Random-weights mode: a model from a configuration and a seed, either written as a
folder (config.json + model.safetensors) or made directly in device memory.

Matrices are N(0, std) and scale vectors (norm weights) 1 + N(0, scale_std); the
reference's own synthetic model (src/l5_model.c:622-680 of AnonymoDGH/gguf2bin) has
all-zero matrices and unit norms, which hides every fault, so it is not imitated.

The generator is counter-based: the value of an element depends on (seed, position of the
tensor in the model's list of tensors, index of the element) and on nothing else.  It is
defined in ``csrc/random_init.cu`` (Philox4x32-10, then Box-Muller in which every
arithmetic step is one IEEE binary32 operation) and exists twice with the same bits: as
that CUDA kernel, which fills a tensor in place in device memory (a model of tens of
gigabytes never touches the disk or the host), and here in numpy for writing a folder
where there is no GPU.  A folder written from a (configuration, seed) therefore loads to
the same model that ``random_tensors_on_device`` makes from them.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import numpy as np
import torch

from .loader import Expected, runtime_dtype
from .safetensors_io import write_safetensors

COUNTER_TAG = 0x6E6F726D          # fourth counter word of this use of Philox ("norm")
_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)
_CHUNK = 1 << 20                  # elements generated at a time on the CPU

_f = np.float32
_LN_COEF = [_f(1.0 / k) for k in (13, 11, 9, 7, 5, 3)]
_SIN_COEF = [_f(-1.0 / 39916800), _f(1.0 / 362880), _f(-1.0 / 5040), _f(1.0 / 120), _f(-1.0 / 6)]
_COS_COEF = [_f(1.0 / 479001600), _f(-1.0 / 3628800), _f(1.0 / 40320), _f(-1.0 / 720), _f(1.0 / 24),
             _f(-0.5)]
_LN2, _HALF_PI = _f(0.6931471805599453), _f(1.5707963267948966)


def _philox_blocks(blocks: np.ndarray, tensor_index: int, seed: int) -> list:
    """Philox4x32-10 for every counter (block lo, block hi, tensor index, tag); four uint64
    arrays holding 32-bit words."""
    c0, c1 = blocks & _MASK, blocks >> np.uint64(32)
    c2 = np.full_like(blocks, np.uint64(tensor_index & 0xFFFFFFFF))
    c3 = np.full_like(blocks, np.uint64(COUNTER_TAG))
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & _MASK, p1 >> np.uint64(32), p1 & _MASK
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return [c0, c1, c2, c3]


def _box_muller(a: np.ndarray, b: np.ndarray):
    """Two standard normals per pair of words, in single float32 operations (numpy rounds
    every float32 operation on its own, which is the definition)."""
    k1 = (a >> np.uint64(8)) + np.uint64(1)
    e = np.frexp(k1.astype(np.float64))[1] - 1                       # k1 = m * 2^e, m in [1, 2)
    m = np.ldexp(k1.astype(np.float32), -e).astype(np.float32)       # exact
    s = (m - _f(1)) / (m + _f(1))
    s2 = s * s
    p = np.full_like(s, _LN_COEF[0])
    for c in _LN_COEF[1:] + [_f(1)]:
        p = p * s2 + c
    ln_u = (e - 24).astype(np.float32) * _LN2 + (_f(2) * s) * p
    r = np.sqrt(_f(-2) * ln_u)
    k2 = b >> np.uint64(8)
    q = (k2 >> np.uint64(22)).astype(np.int64)
    x = ((k2 & np.uint64(0x3FFFFF)).astype(np.float32) * _f(2.0 ** -22)) * _HALF_PI
    x2 = x * x
    ps = np.full_like(x, _SIN_COEF[0])
    for c in _SIN_COEF[1:] + [_f(1)]:
        ps = ps * x2 + c
    sn = x * ps
    pc = np.full_like(x, _COS_COEF[0])
    for c in _COS_COEF[1:] + [_f(1)]:
        pc = pc * x2 + c
    cos = np.choose(q, [pc, -sn, -pc, sn])
    sin = np.choose(q, [sn, pc, -sn, -pc])
    return r * cos, r * sin


def normal_values(n: int, seed: int, tensor_index: int, first: int = 0) -> np.ndarray:
    """Elements first .. first+n-1 of the standard-normal stream of (seed, tensor index),
    float32.  ``first`` must be a multiple of four."""
    if first % 4:
        raise ValueError("normal_values: first must be a multiple of 4")
    n_blocks = -(-n // 4)
    blocks = np.arange(first // 4, first // 4 + n_blocks, dtype=np.uint64)
    w = _philox_blocks(blocks, tensor_index, int(seed))
    z = np.empty((n_blocks, 4), dtype=np.float32)
    z[:, 0], z[:, 1] = _box_muller(w[0], w[1])
    z[:, 2], z[:, 3] = _box_muller(w[2], w[3])
    return z.reshape(-1)[:n]


def random_tensor(e: Expected, seed: int, index: int, dtype: torch.dtype,
                  std: float, scale_std: float) -> torch.Tensor:
    """The tensor at position ``index`` of a model's list, made on the CPU."""
    n = 1
    for d in e.shape:
        n *= int(d)
    if e.init not in ("matrix", "scale"):
        raise ValueError(f"unknown init kind {e.init!r}")
    out = torch.empty(n, dtype=dtype)
    for first in range(0, n, _CHUNK):
        z = normal_values(min(_CHUNK, n - first), seed, index, first)
        v = _f(scale_std) * z + _f(1) if e.init == "scale" else _f(std) * z
        out[first:first + len(v)] = torch.from_numpy(v).to(dtype)
    return out.view(tuple(e.shape))


def fill_random_on_device(out: torch.Tensor, e: Expected, seed: int, index: int, std: float,
                          scale_std: float) -> None:
    """The same tensor, made in place in device memory by the CUDA kernel."""
    from .. import kernels
    if e.init not in ("matrix", "scale"):
        raise ValueError(f"unknown init kind {e.init!r}")
    kernels.philox_normal(out, seed, index, e.init == "scale", scale_std if e.init == "scale" else std)


def random_tensors_on_device(expected: Mapping[str, Expected], seed: int, storage: torch.dtype,
                             compute: torch.dtype, device, std: float = 0.02,
                             scale_std: float = 0.1) -> dict:
    """name -> tensor on ``device`` for every non-optional expected tensor: generated in the
    storage dtype (what a written folder would hold), kept in the dtype the loader would
    give it under ``compute``."""
    tensors = {}
    for i, (name, e) in enumerate(expected.items()):
        if e.optional:
            continue
        t = torch.empty(tuple(e.shape), dtype=storage, device=device)
        fill_random_on_device(t, e, seed, i, std, scale_std)
        tensors[name] = t.to(runtime_dtype(storage, compute))
    return tensors


def write_random_model(folder, config: Mapping, seed: int, dtype: str = "bfloat16",
                       std: float = 0.02, scale_std: float = 0.1,
                       expected: Mapping[str, Expected] | None = None,
                       on_device: bool | None = None) -> Path:
    """Writes ``folder/config.json`` and ``folder/model.safetensors``.  ``dtype`` is the
    storage type of every tensor ("bfloat16" or "float32").  ``expected`` defaults to the
    tensors of the model that ``config`` describes.  Tensors are made by the CUDA kernel when
    a GPU is there (a model of several gigabytes takes seconds), else on the CPU (``on_device``
    forces one or the other); the bits are the same."""
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
    if on_device is None:
        on_device = torch.cuda.is_available()

    def make(e, i):
        if not on_device:
            return random_tensor(e, seed, i, tdtype, std, scale_std)
        t = torch.empty(tuple(e.shape), dtype=tdtype, device="cuda")
        fill_random_on_device(t, e, seed, i, std, scale_std)
        return t.cpu()

    items = []
    for i, (name, e) in enumerate(expected.items()):
        if e.optional:
            continue
        items.append((name, tuple(e.shape), tdtype, (lambda e=e, i=i: make(e, i))))
    write_safetensors(folder / "model.safetensors", items)
    return folder
