"""Shared by the tests: the tiny configurations, model folders in temporary places, the
plain implementation's logits, and the comparison rules."""
from __future__ import annotations

import functools
import tempfile
from pathlib import Path

import numpy as np

from plain import qwen3_plain as P

# Two tiny configurations that differ in every size and option, plus two whose head
# sizes (64, 128) are the ones the tensor-core kernels take.
TINY = {
    "a": dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
              num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
              vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=64),
    "b": dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=224,
              num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
              vocab_size=311, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
              max_position_embeddings=128),
    "c": dict(architectures=["Qwen3ForCausalLM"], hidden_size=192, intermediate_size=328,
              num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
              vocab_size=533, rope_theta=5e5, rms_norm_eps=1e-6, tie_word_embeddings=False,
              max_position_embeddings=640),
    "d": dict(architectures=["Qwen3ForCausalLM"], hidden_size=256, intermediate_size=520,
              num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=1, head_dim=128,
              vocab_size=1000, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=512),
}
SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3}

_tmp_root = None


def tmp_root() -> Path:
    global _tmp_root
    if _tmp_root is None:
        _tmp_root = tempfile.TemporaryDirectory(prefix="g2b_tests_")
    return Path(_tmp_root.name)


@functools.lru_cache(maxsize=None)
def model_folder(name: str, storage: str = "float32") -> Path:
    """A model folder of a tiny configuration with random weights, made once per run."""
    from gguf2bin_b200.weights import write_random_model
    folder = tmp_root() / f"tiny_{name}_{storage}"
    write_random_model(folder, TINY[name], SEEDS[name], storage)
    return folder


@functools.lru_cache(maxsize=None)
def plain_model(name: str, storage: str = "float32"):
    return P.read_model_folder(model_folder(name, storage))


def random_tokens(name: str, n: int, seed: int) -> list[int]:
    rng = np.random.default_rng(1000 + seed)
    return rng.integers(0, TINY[name]["vocab_size"], n).tolist()


_plain_cache: dict = {}


def plain_logits(name: str, storage: str, tokens) -> np.ndarray:
    key = (name, storage, tuple(tokens))
    if key not in _plain_cache:
        cfg, W = plain_model(name, storage)
        _plain_cache[key] = P.forward(cfg, W, list(tokens), np.float32)
    return _plain_cache[key]


def tolerance(dtype: str, ref: np.ndarray) -> float:
    """float32: 1e-5 of the logit scale (the plain implementation itself is within 5e-7
    of the reference's C).  bfloat16: activations between kernels carry 8 bits, 2^-8
    relative per rounding; eight roundings' worth of the logit scale."""
    scale = max(1.0, float(np.abs(ref).max()))
    return (1e-5 if dtype == "float32" else 8 * 2.0 ** -8) * scale


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str) -> None:
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - ref)
    tol = tolerance(dtype, ref)
    if err.max() > tol:
        pos = np.unravel_index(err.argmax(), err.shape)
        first_bad = int(np.nonzero(err.max(axis=-1) > tol)[0][0]) if err.ndim == 2 else -1
        raise AssertionError(f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at {pos}; first "
                             f"row over tolerance: {first_bad}")
