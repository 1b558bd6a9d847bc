"""The plain implementation against logits that the reference's own C code produced
(tests/golden/make_golden.py built src/l1..l6 of AnonymoDGH/gguf2bin here on the CPU and
ran model_forward token by token)."""
import numpy as np
import pytest

from golden.make_golden import CASES, HERE, case_weights
from plain import qwen3_plain as P


@pytest.mark.parametrize("name", sorted(CASES))
def test_plain_matches_reference_c(name):
    cfg, W, ids = case_weights(name)
    golden = np.load(HERE / f"{name}_logits.npy")
    got = P.forward(cfg, W, ids, np.float32)
    assert got.shape == golden.shape
    assert np.abs(got - golden).max() < 2e-6
    assert (got.argmax(1) == golden.argmax(1)).all()


def test_plain_parts_against_float64():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 80)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(80)).astype(np.float32)
    a = P.rmsnorm(x, w, 1e-6, np.float32)
    b = P.rmsnorm(x, w, 1e-6, np.float64)
    assert np.abs(a - b).max() < 1e-5
    # rotation keeps the norm of every pair and is the identity at position 0
    q = rng.standard_normal((3, 2, 16)).astype(np.float32)
    r = P.rope_neox(q, [0, 5, 9], 1e4, np.float64)
    assert np.allclose(r[0], q[0])
    assert np.allclose((r ** 2).sum(-1), (q.astype(np.float64) ** 2).sum(-1))
    # a window as long as the sequence is full attention
    k = rng.standard_normal((7, 1, 16)).astype(np.float32)
    v = rng.standard_normal((7, 1, 16)).astype(np.float32)
    qq = rng.standard_normal((7, 2, 16)).astype(np.float32)
    assert np.allclose(P.causal_attention(qq, k, v, np.float64),
                       P.causal_attention(qq, k, v, np.float64, window=7))
    # position 0 attends to itself only
    assert np.allclose(P.causal_attention(qq, k, v, np.float64)[0], np.repeat(v[0], 2, 0))


def test_plain_samplers():
    l = np.array([0.1, 2.0, 2.0, -1.0], np.float32)
    assert P.greedy(l) == 1
    i, cdf = P.sample_temperature(l, 1.0, 0.0)
    assert i == 0
    assert P.sample_temperature(l, 1.0, 1.0)[0] == 3
    # top_k 1 is greedy whatever r is; penalty lowers a recent positive logit
    assert P.sample_advanced(l, 1.0, 1, 1.0, 1.0, [], 0.99)[0] == 1
    assert P.sample_advanced(l, 0.0, 0, 1.0, 2.0, [1], 0.5)[0] == 2
    out = P.apply_repeat_penalty(l, 2.0, [3, 3, 0])
    assert np.allclose(out, [0.05, 2.0, 2.0, -2.0])
