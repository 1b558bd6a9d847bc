"""Random weights made on the device: the kernel against the plain definition bit for bit,
and a model made in device memory against the same model written to a folder and loaded."""
import numpy as np
import pytest
import torch

from helpers import TINY, random_tokens, tmp_root
from plain import philox_normal_plain as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,std", [("matrix", 0.02), ("scale", 0.1)])
def test_kernel_follows_the_plain_definition(dtype, kind, std):
    from gguf2bin_b200 import kernels
    for seed, tensor, n in ((0, 0, 1), (9, 3, 6), (2 ** 35 + 1, 291, 203)):
        out = torch.full((n + 4,), 7.0, dtype=dtype, device=DEV)
        kernels.philox_normal(out[:n], seed, tensor, kind == "scale", std)
        got = out.cpu()
        assert (got[n:] == 7.0).all(), "the kernel wrote past the tensor"
        want = [Q.value(seed, tensor, i, kind, std) for i in range(n)]
        if dtype == torch.float32:
            assert np.array_equal(got[:n].numpy().view(np.uint32), np.array(want, np.float32).view(np.uint32))
        else:
            bits = got[:n].view(torch.int16).numpy().astype(np.uint16)
            assert [int(b) for b in bits] == [Q.to_bfloat16_bits(v) for v in want]


def test_kernel_equals_the_cpu_generator_on_a_large_tensor():
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.weights import Expected, random_tensor
    n = (1 << 21) + 3
    out = torch.empty(n, dtype=torch.float32, device=DEV)
    kernels.philox_normal(out, 123456789, 17, False, 0.02)
    ref = random_tensor(Expected((n,)), 123456789, 17, torch.float32, 0.02, 0.1)
    assert torch.equal(out.cpu(), ref)
    z = out.double() / 0.02
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1) < 0.01


@pytest.mark.parametrize("name,dtype,storage", [("b", "float32", "float32"), ("c", "bfloat16", "bfloat16"),
                                                ("a", "float32", "bfloat16")])
def test_a_model_made_on_the_device_is_the_model_synth_writes(name, dtype, storage):
    """Same (configuration, seed): a folder written by the CPU generator and loaded, and a
    model made in device memory, hold the same tensors and give the same logits."""
    from gguf2bin_b200.engine import Engine, Model, StepEntry
    from gguf2bin_b200.weights.random_init import write_random_model
    folder = tmp_root() / f"synth_{name}_{storage}"
    write_random_model(folder, TINY[name], 42, storage, on_device=False)
    loaded = Model.from_folder(folder, dtype=dtype)
    made = Model.random(TINY[name], 42, dtype=dtype, storage=storage)
    a, b = list(loaded._all_weights()), list(made._all_weights())
    assert len(a) == len(b) > 10
    for x, y in zip(a, b):
        assert x.dtype == y.dtype and torch.equal(x, y)
    toks = random_tokens(name, 23, 1)
    outs = []
    for m in (loaded, made):
        eng = Engine(m, max_tokens=256)
        s = eng.open_sequence()
        outs.append(eng.step([StepEntry(s, toks, range(len(toks)))]).clone())
    assert torch.equal(outs[0], outs[1])


def test_llm_random_generates():
    from gguf2bin_b200.api import LLM
    llm = LLM.random(TINY["d"], seed=3, dtype="bfloat16", max_tokens=512)
    again = LLM.random(TINY["d"], seed=3, dtype="bfloat16", max_tokens=512)
    other = LLM.random(TINY["d"], seed=4, dtype="bfloat16", max_tokens=512)
    kw = dict(n=8, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    p = [random_tokens("d", 12, 2)]
    assert llm.generate(p, **kw)[0].tokens == again.generate(p, **kw)[0].tokens
    assert llm.generate(p, **kw)[0].tokens != other.generate(p, **kw)[0].tokens
