"""The allocation-free decode attention entry point (csrc/attn_decode_noalloc.h), called
through its exported C symbol.

Some users of the library cannot allocate device memory when they call it (a plugin inside
a process whose allocator owns the whole GPU; a loop that cannot take the synchronisation
an allocation may bring), so this entry point keeps its scratch in an array inside the
shared object.  The test checks its output two ways: against the plain implementation's
attention (the arithmetic is right), and bit for bit against the ordinary entry point of
the SAME shared object given scratch that the test allocates (the only difference between
the two is where the scratch lives).

The file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It passes alone in a fresh process as well as after the
other tests: it builds its own inputs and loads the shared object itself.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD, PAGE = 128, 64


def _library():
    """The object as ``build()`` ships it: the head size is its only define."""
    from gguf2bin_b200.csrc import build
    lib = ctypes.CDLL(str(build.compile_unit("attn_decode_noalloc.cu", (f"HD={HD}",))))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.g2b_attn_decode_noalloc.restype = ci
    lib.g2b_attn_decode_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci,
                                            ctypes.c_float, ci, vp]
    lib.g2b_attn_decode.restype = ci
    lib.g2b_attn_decode.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci,
                                    ctypes.c_float, ci, vp, vp, vp]
    lib.g2b_last_error.restype = ctypes.c_char_p
    lib.g2b_attn_decode_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    lib.g2b_attn_decode_chunk_keys.restype = ci
    return lib


def _case(lens, nh, nkv, seed):
    """A paged bfloat16 cache (pages shuffled, junk where no key lies) holding random keys
    and values for sequences of the given lengths; one query token at the end of each."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-l // PAGE) for l in lens]
    n_pages = sum(pages_per) + 2
    cache = torch.randn(n_pages, 2, nkv, PAGE, HD, generator=g).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lens), max(pages_per), dtype=torch.int32)
    keys, values, nxt = [], [], 0
    for b, l in enumerate(lens):
        K = torch.randn(l, nkv, HD, generator=g).to(torch.bfloat16)
        V = torch.randn(l, nkv, HD, generator=g).to(torch.bfloat16)
        for p in range(pages_per[b]):
            pg = perm[nxt]
            nxt += 1
            table[b, p] = pg
            n = min(PAGE, l - p * PAGE)
            cache[pg, 0, :, :n] = K[p * PAGE:p * PAGE + n].transpose(0, 1)
            cache[pg, 1, :, :n] = V[p * PAGE:p * PAGE + n].transpose(0, 1)
        keys.append(K.float().numpy())
        values.append(V.float().numpy())
    q = torch.randn(len(lens), nh * HD, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    return q, cache.to(DEV), table.to(DEV), pos, seq, keys, values


def _plain(q, keys, values, nh, window):
    """The last row of the plain causal attention of each sequence."""
    rows = []
    for b, (K, V) in enumerate(zip(keys, values)):
        qfull = np.zeros((len(K), nh, HD), np.float32)
        qfull[-1] = q[b].float().cpu().numpy().reshape(nh, HD)
        rows.append(P.causal_attention(qfull, K, V, np.float32, window=window)[-1].reshape(-1))
    return np.stack(rows)


def _args(q, out, cache, table, pos, seq, nh, nkv, window):
    return (q.data_ptr(), out.data_ptr(), cache.data_ptr(), pos.data_ptr(), seq.data_ptr(),
            table.data_ptr(), table.shape[1], q.shape[0], nh, nkv, HD, PAGE, window,
            1 / math.sqrt(HD), table.shape[1] * PAGE)


def test_two_calls_in_a_row_match_the_plain_attention_and_the_ordinary_entry_point():
    lib = _library()
    assert lib.g2b_attn_decode_noalloc_scratch_bytes() == 16 * 1024 * 1024
    chunk = lib.g2b_attn_decode_chunk_keys()
    stream = torch.cuda.current_stream().cuda_stream
    # the second call is smaller and differently shaped: whatever the first left in the
    # shared scratch must not leak into it
    for i, (lens, nh, nkv, window) in enumerate([([700, 1, 257, 64, 1025], 16, 8, 0),
                                                 ([300, 90], 10, 2, 100)]):
        q, cache, table, pos, seq, keys, values = _case(lens, nh, nkv, seed=90 + i)
        # the ordinary entry point of the same object, with scratch allocated here
        n_chunks = -(-table.shape[1] * PAGE // chunk)
        part_o = torch.empty(len(lens) * nh * n_chunks * HD, dtype=torch.float32, device=DEV)
        part_ml = torch.empty(len(lens) * nh * n_chunks * 2, dtype=torch.float32, device=DEV)
        same = torch.empty_like(q)
        rc = lib.g2b_attn_decode(*_args(q, same, cache, table, pos, seq, nh, nkv, window),
                                 part_o.data_ptr(), part_ml.data_ptr(), stream)
        assert rc == 0, lib.g2b_last_error().decode()
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        got = torch.empty_like(q)
        rc = lib.g2b_attn_decode_noalloc(*_args(q, got, cache, table, pos, seq, nh, nkv, window), stream)
        assert rc == 0, lib.g2b_last_error().decode()
        torch.cuda.synchronize()
        if i == 1:      # by the second call the object's code and array are resident
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        assert torch.equal(got, same), f"call {i}: differs from the ordinary entry point of the same object"
        want = _plain(q, keys, values, nh, window)
        tol = 2.0 ** -7 * max(1.0, float(np.abs(want).max()))        # as tests/test_gpu_kernels.py
        assert np.isfinite(got.float().cpu().numpy()).all()
        assert np.abs(got.float().cpu().numpy() - want).max() <= tol, f"call {i}: differs from the plain attention"


def test_requests_beyond_the_array_are_refused():
    lib = _library()
    q, cache, table, pos, seq, _, _ = _case([64] * 4, 16, 8, seed=5)
    out = torch.full_like(q, 3.0)
    chunk = lib.g2b_attn_decode_chunk_keys()
    # 4 tokens x 16 heads x 512 chunks x 130 floats = 17 MB > 16 MiB
    rc = lib.g2b_attn_decode_noalloc(q.data_ptr(), out.data_ptr(), cache.data_ptr(), pos.data_ptr(),
                                     seq.data_ptr(), table.data_ptr(), table.shape[1], 4, 16, 8, HD,
                                     PAGE, 0, 0.1, 512 * chunk, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.g2b_last_error().decode()
    assert "16777216" in msg and "scratch" in msg
    torch.cuda.synchronize()
    assert (out == 3.0).all(), "a refused call must launch nothing"
    # the limits the header states for 16 heads of 128: 8 tokens at 64,512 keys fit, one chunk more does not
    per_chunk = 16 * (HD + 2) * 4
    assert 8 * per_chunk * (64512 // 256) <= 16 * 1024 * 1024 < 8 * per_chunk * (64512 // 256 + 1)
    assert 64 * per_chunk * (7936 // 256) <= 16 * 1024 * 1024 < 64 * per_chunk * (7936 // 256 + 1)
