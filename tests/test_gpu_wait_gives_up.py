"""The give-up path of the tcgen05 kernels' bounded waits, made to run without harming
anything: a build of the same sources in which the copy-issuing role issues nothing and the
limit of a wait is 4,096 polls (csrc/tc_common.cuh).  No copy is in flight and no product is
issued, so every waiting role runs out of polls within microseconds, records its code in the
status word, the tensor memory is freed and the kernel returns by itself.  The host then
reads the status as a ``KernelError``, and the next ordinary launch in the same process is
right: the context is intact and the status word is clear again."""
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("what,M,N,K,bn,stages,mode", [
    ("one tile per CTA", 200, 1000, 1032, 128, 3, False),
    ("persistent", 1500, 2048, 1024, 256, 4, True),
    ("pairs of CTAs", 600, 1024, 520, 256, 6, 2),
    ("K split over a cluster", 40, 4096, 4096, 0, 0, 3),
])
def test_product_whose_copies_never_come(what, M, N, K, bn, stages, mode):
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.csrc.units import WAITS_RUN_OUT
    from gguf2bin_b200.kernels import KernelError
    kernels_bf16.check_status()                                  # nothing pending from earlier tests
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=1), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=2)
    out = torch.zeros(M, N, device=DEV)
    kernels_bf16._gemm_tc(a, w, out, kernels_bf16.EPI_STORE_F32, bn, stages, mode, defines=WAITS_RUN_OUT)
    torch.cuda.synchronize()                                     # the kernel returned by itself
    with pytest.raises(KernelError, match=r"gemm_tc.*(MMA issuer|epilogue|a CTA of a pair).*gave up waiting"):
        kernels_bf16.check_status()
    kernels_bf16.check_status()                                  # reading the status cleared it
    # the same product by the library's own build, right after, in the same context
    kernels_bf16._gemm_tc(a, w, out, kernels_bf16.EPI_STORE_F32, bn, stages, mode)
    kernels_bf16.check_status()
    ref = a.double() @ w.double().T
    assert (out.double() - ref).abs().max().item() < 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("split", [False, True])
def test_prompt_attention_whose_copies_never_come(split):
    from types import SimpleNamespace
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.csrc.units import WAITS_RUN_OUT
    from gguf2bin_b200.kernels import KernelError
    nh, nkv, hd, ps, T = 4, 2, 128, 64, 200
    kernels_bf16.check_status()
    g = torch.Generator().manual_seed(5)
    K, V = (torch.randn(T, nkv, hd, generator=g).to(torch.bfloat16) for _ in range(2))
    n_pages = -(-T // ps)
    cache = torch.zeros(n_pages + 1, 2, nkv, ps, hd, dtype=torch.bfloat16)
    for p in range(n_pages):
        n = min(ps, T - p * ps)
        cache[p + 1, 0, :, :n] = K[p * ps:p * ps + n].transpose(0, 1)
        cache[p + 1, 1, :, :n] = V[p * ps:p * ps + n].transpose(0, 1)
    cache = cache.to(DEV)
    table = torch.arange(1, n_pages + 1, dtype=torch.int32, device=DEV).view(1, -1)
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=6)
    tiles = torch.tensor([[0, 128, T - 128, 128], [0, 0, 128, 0]], dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(attn_tiles_wide=tiles, n_attn_tiles_wide=2, page_table=table)
    out = torch.zeros_like(q)
    kernels_bf16.attn_prefill_tc(q, out, cache, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd), defines=WAITS_RUN_OUT,
                                 split=split)
    torch.cuda.synchronize()
    with pytest.raises(KernelError, match=r"attn_prefill_tc.*gave up waiting"):
        kernels_bf16.check_status()
    kernels_bf16.attn_prefill_tc(q, out, cache, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd), split=split)
    kernels_bf16.check_status()
    ref = P.causal_attention(q.float().cpu().numpy().reshape(T, nh, hd), K.float().numpy(), V.float().numpy(),
                             np.float32)
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    assert np.abs(got - ref).max() <= 2.0 ** -7 * max(1.0, np.abs(ref).max())


def test_the_engine_reports_a_wait_that_gave_up():
    """A status word that a kernel left set surfaces as a ``KernelError`` at the engine's next
    point of synchronisation, so tokens or logits of that launch are never handed on."""
    from helpers import model_folder, random_tokens
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.api import LLM
    from gguf2bin_b200.kernels import KernelError
    llm = LLM(model_folder("d", "bfloat16"), dtype="bfloat16", max_tokens=512)
    kw = dict(n=4, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    llm.generate([random_tokens("d", 40, 1)], **kw)
    kernels_bf16._status_word(DEV).fill_(2)                      # as a kernel's issuer would leave it
    with pytest.raises(KernelError, match="gave up waiting"):
        llm.generate([random_tokens("d", 40, 1)], **kw)
    assert llm.engine.cache.table.slots.n_held == 0             # the failed call gave everything back
    assert len(llm.generate([random_tokens("d", 40, 1)], **kw)[0].tokens) == 4
