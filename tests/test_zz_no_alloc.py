"""The allocation-free decode attention entry point (csrc/attn_decode_noalloc.h), called
through its exported C symbol, against the ordinary entry point.

The file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test.  It passes alone in a fresh process as well as after the
other tests: it builds its own inputs and loads the shared object itself.
"""
import ctypes
import math
from types import SimpleNamespace

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HD, PAGE = 128, 64


def _library():
    from gguf2bin_b200.csrc import build
    lib = ctypes.CDLL(str(build.compile_unit("attn_decode_noalloc.cu", (f"HD={HD}",))))
    f = lib.g2b_attn_decode_noalloc
    f.restype = ctypes.c_int
    vp, ci = ctypes.c_void_p, ctypes.c_int
    f.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ctypes.c_float, ci, vp]
    lib.g2b_last_error.restype = ctypes.c_char_p
    lib.g2b_attn_decode_noalloc_scratch_bytes.restype = ctypes.c_ulonglong
    return lib


def _case(lens, nh, nkv, seed):
    """A paged bfloat16 cache with random keys and values for sequences of the given
    lengths (pages shuffled), one query token at the end of each."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-l // PAGE) for l in lens) + 2
    cache = (torch.randn(n_pages, 2, nkv, PAGE, HD, generator=g)).to(torch.bfloat16).to(DEV)
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(len(lens), max(-(-l // PAGE) for l in lens), dtype=torch.int32)
    nxt = 0
    for b, l in enumerate(lens):
        for p in range(-(-l // PAGE)):
            table[b, p] = perm[nxt]
            nxt += 1
    q = torch.randn(len(lens), nh * HD, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    return q, cache, table.to(DEV), pos, seq


def _ordinary(q, cache, table, pos, seq, nh, nkv, window):
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.engine.workspace import Workspace
    out = torch.empty_like(q)
    ctx = SimpleNamespace(tok_pos=pos, tok_seq=seq, page_table=table, workspace=Workspace(DEV),
                          max_kv_len=table.shape[1] * PAGE, all_single=True)
    kernels_bf16.attn_decode(q, out, cache, ctx, nh, nkv, HD, PAGE, window, 1 / math.sqrt(HD))
    return out


def _no_alloc(lib, q, cache, table, pos, seq, nh, nkv, window):
    out = torch.empty_like(q)
    rc = lib.g2b_attn_decode_noalloc(
        q.data_ptr(), out.data_ptr(), cache.data_ptr(), pos.data_ptr(), seq.data_ptr(),
        table.data_ptr(), table.shape[1], q.shape[0], nh, nkv, HD, PAGE, window,
        1 / math.sqrt(HD), table.shape[1] * PAGE, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.g2b_last_error().decode()
    return out


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    lib = _library()
    assert lib.g2b_attn_decode_noalloc_scratch_bytes() == 16 * 1024 * 1024
    # the second call is smaller and differently shaped: whatever the first left in the
    # shared scratch must not leak into it
    for i, (lens, nh, nkv, window) in enumerate([([700, 1, 257, 64, 1025], 16, 8, 0),
                                                 ([300, 90], 10, 2, 100)]):
        q, cache, table, pos, seq = _case(lens, nh, nkv, seed=90 + i)
        want = _ordinary(q, cache, table, pos, seq, nh, nkv, window)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        got = _no_alloc(lib, q, cache, table, pos, seq, nh, nkv, window)
        torch.cuda.synchronize()
        if i == 1:      # by the second call the object's code and array are resident
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the free device memory"
        assert torch.isfinite(got.float()).all()
        tol = 2.0 ** -7 * max(1.0, want.float().abs().max().item())   # as tests/test_gpu_kernels.py
        assert (got.float() - want.float()).abs().max().item() <= tol, f"call {i}"


def test_requests_beyond_the_array_are_refused():
    lib = _library()
    q, cache, table, pos, seq = _case([64] * 4, 16, 8, seed=5)
    out = torch.full_like(q, 3.0)
    # 4 tokens x 16 heads x 512 chunks of 256 keys x 130 floats = 17 MB > 16 MiB
    rc = lib.g2b_attn_decode_noalloc(q.data_ptr(), out.data_ptr(), cache.data_ptr(), pos.data_ptr(),
                                     seq.data_ptr(), table.data_ptr(), table.shape[1], 4, 16, 8, HD,
                                     PAGE, 0, 0.1, 512 * 256, torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    msg = lib.g2b_last_error().decode()
    assert "16777216" in msg and "scratch" in msg
    torch.cuda.synchronize()
    assert (out == 3.0).all(), "a refused call must launch nothing"
