"""Shared by the tests: the tiny configurations, model folders in temporary places, the
plain implementation's logits, and the comparison rules."""
from __future__ import annotations

import functools
import os
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
    # a vocabulary large enough for the samplers that cut a row into slices (8,192 entries and more),
    # and no multiple of four: every second row of logits starts off a 16-byte boundary
    "e": dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=96,
              num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=32,
              vocab_size=8209, rope_theta=1e4, rms_norm_eps=1e-6, tie_word_embeddings=True,
              max_position_embeddings=96),
}
SEEDS = {"a": 0, "b": 1, "c": 2, "d": 3, "e": 4}

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


# bfloat16 bounds, set from what was measured over every comparison of the GPU suite
# (G2B_ERROR_REPORT): the worst max |diff| was 0.0093 of max |logit| in the models of the
# architecture (0.0139 in a toy model whose head scales the logits by nine) and the worst rms
# diff 0.0082 of the logits' rms, medians 0.0052 and 0.0049.  The bounds are two to three
# times the worst seen, relative to the logits themselves (no floor): a systematic error of
# one bfloat16 rounding of the logit scale shows in the rms bound before it shows in the max.
BF16_MAX_REL = 0.028
BF16_RMS_REL = 0.016
F32_REL = 1e-5


def tolerance(dtype: str, ref: np.ndarray) -> float:
    """The bound on max |diff|.  float32: 1e-5 of the logit scale (the plain implementation
    itself is within 5e-7 of the reference's C; the worst seen here is 3e-6).  bfloat16:
    ``BF16_MAX_REL`` of the largest logit."""
    top = float(np.abs(ref).max())
    return F32_REL * max(1.0, top) if dtype == "float32" else BF16_MAX_REL * max(top, 1e-3)


def _report(what: str, dtype: str, got: np.ndarray, ref: np.ndarray) -> None:
    """With G2B_ERROR_REPORT=<file> every comparison appends a line: what, dtype, max |diff|,
    rms diff, max |ref|, rms ref, rows, rows whose argmax agrees (as the reference's
    tools/kvtest.c:26-47 reports max abs delta, rmse and argmax agreement)."""
    path = os.environ.get("G2B_ERROR_REPORT")
    if not path:
        return
    d = (got - ref).astype(np.float64)
    rows = got.reshape(-1, got.shape[-1])
    agree = int((rows.argmax(-1) == ref.reshape(rows.shape).argmax(-1)).sum())
    with open(path, "a") as f:
        f.write(f"{what}\t{dtype}\t{np.abs(d).max():.4e}\t{np.sqrt((d ** 2).mean()):.4e}\t"
                f"{np.abs(ref).max():.4e}\t{np.sqrt((ref.astype(np.float64) ** 2).mean()):.4e}\t"
                f"{rows.shape[0]}\t{agree}\n")


def assert_close(got: np.ndarray, ref: np.ndarray, dtype: str, what: str) -> None:
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    _report(what, dtype, got, ref)
    err = np.abs(got - ref)
    tol = tolerance(dtype, ref)
    if err.max() > tol:
        pos = np.unravel_index(err.argmax(), err.shape)
        first_bad = int(np.nonzero(err.max(axis=-1) > tol)[0][0]) if err.ndim == 2 else -1
        raise AssertionError(f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at {pos}; first "
                             f"row over tolerance: {first_bad}")
    # the three figures the reference's own comparison tool reports (tools/kvtest.c:26-47):
    # max abs difference (above), rms difference, and agreement of the argmax
    rms_err = float(np.sqrt((err.astype(np.float64) ** 2).mean()))
    rms_ref = float(np.sqrt((ref.astype(np.float64) ** 2).mean()))
    rms_tol = (F32_REL if dtype == "float32" else BF16_RMS_REL) * max(rms_ref, 1e-3)
    assert rms_err <= rms_tol, f"{what}: rms diff {rms_err:.3e} > {rms_tol:.3e} (rms of the logits {rms_ref:.3e})"
    if got.ndim == 2:
        top2 = np.sort(ref, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 2 * err.max(axis=-1)        # the row's own error cannot flip these
        wrong = np.nonzero(clear & (got.argmax(-1) != ref.argmax(-1)))[0]
        assert len(wrong) == 0, f"{what}: argmax differs in rows {wrong[:5].tolist()}"
