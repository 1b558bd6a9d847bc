"""The engine at the layer sizes of the benchmark configurations (Qwen3-0.6B, 8B, 14B) with
few layers, against the plain implementation: an unequal batch of prompts in one step, then
a few single-token steps.  The 0.6B case keeps the real vocabulary (151,936, tied); the two
larger ones use a small vocabulary so that the files stay small (the vocabulary is not a
layer size)."""
import numpy as np
import pytest

from helpers import assert_close, tmp_root
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu

SIZES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=2, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=1, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, vocab_size=1000, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=1, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, vocab_size=1000, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name,dtype", [("0.6b", "bfloat16"), ("0.6b", "float32"), ("8b", "bfloat16"),
                                        ("14b", "bfloat16")])
def test_layer_sizes(name, dtype):
    from gguf2bin_b200.engine import Engine, Model, StepEntry
    from gguf2bin_b200.weights import write_random_model
    cfg = dict(architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=40960, **SIZES[name])
    folder = write_random_model(tmp_root() / f"sizes_{name}", cfg, seed=11, dtype="bfloat16")
    pcfg, W = P.read_model_folder(folder)
    rng = np.random.default_rng(5)
    reqs = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (70, 9, 133)]
    n_dec = 3
    eng = Engine(Model.from_folder(folder, dtype=dtype), max_tokens=1024)
    seqs = [eng.open_sequence() for _ in reqs]
    heads = [len(t) - n_dec for t in reqs]
    got = [[] for _ in reqs]
    out = eng.step([StepEntry(s, t[:h], [h - 2, h - 1]) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
    for j in range(len(reqs)):
        got[j].append(out[2 * j:2 * j + 2])
    for d in range(n_dec):
        out = eng.step([StepEntry(s, [t[h + d]], [0]) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
        for j in range(len(reqs)):
            got[j].append(out[j:j + 1])
    for j, toks in enumerate(reqs):
        ref = P.forward(pcfg, W, toks, np.float32)[heads[j] - 2:]
        assert_close(np.concatenate(got[j]), ref, dtype, f"{name}/{dtype} request {j}")
    if dtype == "bfloat16":
        from gguf2bin_b200 import kernels_bf16
        kernels_bf16.check_status()


SIZES["0.6b-small-vocab"] = dict(SIZES["0.6b"], vocab_size=1000)


@pytest.mark.parametrize("name,n_requests", [("8b", 12), ("14b", 40), ("0.6b-small-vocab", 12),
                                             ("0.6b-small-vocab", 24), ("0.6b-small-vocab", 40),
                                             ("0.6b-small-vocab", 64)])
def test_layer_sizes_in_a_wider_batch(name, n_requests):
    """The same at 12 to 64 sequences: from 9 rows on the products of the larger widths run on
    the kernel that splits K over a cluster (32 and 64 rows of activations per CTA), and from
    17 rows on so do most products of the small model's layers (K = 1,024 and 3,072), which
    is the route the benchmark's batch of 64 takes.  Short prompts, so that the plain
    implementation stays quick."""
    from gguf2bin_b200.engine import Engine, Model, StepEntry
    from gguf2bin_b200.weights import write_random_model
    from gguf2bin_b200 import kernels_bf16
    cfg = dict(architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6,
               max_position_embeddings=40960, **SIZES[name])
    folder = write_random_model(tmp_root() / f"sizes_wide_{name}", cfg, seed=12, dtype="bfloat16")
    pcfg, W = P.read_model_folder(folder)
    rng = np.random.default_rng(6)
    reqs = [rng.integers(0, cfg["vocab_size"], 2 + i % 4).tolist() for i in range(n_requests)]
    eng = Engine(Model.from_folder(folder, dtype="bfloat16"), max_tokens=64 * n_requests)
    seqs = [eng.open_sequence() for _ in reqs]
    heads = [len(t) - 1 for t in reqs]
    out = eng.step([StepEntry(s, t[:h], [h - 1]) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
    dec = eng.step([StepEntry(s, [t[h]], [0]) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
    kernels_bf16.check_status()
    for j, toks in enumerate(reqs):
        ref = P.forward(pcfg, W, toks, np.float32)[heads[j] - 1:]
        assert_close(np.stack([out[j], dec[j]]), ref, "bfloat16", f"{name} request {j} of {n_requests}")
