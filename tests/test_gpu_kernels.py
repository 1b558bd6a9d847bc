"""Each kernel alone against a plain float32 computation in torch/numpy, at sizes other
than the engine's: widths that are no power of two, odd row counts, shuffled pages."""
import math

import numpy as np
import pytest
import torch

from plain import philox_plain, qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(dtype):
    from gguf2bin_b200 import kernels
    table = rnd(311, 100, dtype=dtype)
    ids = torch.tensor([0, 310, 5, 5, 17], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 100, device=DEV)
    kernels.embed_rows(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("H", [100, 64, 1030, 128, 1024, 1028, 2560, 4096, 5120, 8192, 8200])
@pytest.mark.parametrize("odtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(H, odtype):
    from gguf2bin_b200 import kernels
    x, w = rnd(7, H, seed=1), 1 + 0.1 * rnd(H, seed=2)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    for r in (None, rows):
        n = 7 if r is None else 3
        out = torch.empty(n, H, dtype=odtype, device=DEV)
        kernels.rmsnorm(x, w, 1e-5, out, r)
        xs = x if r is None else x[r.long()]
        ref = P.rmsnorm(xs.cpu().numpy(), w.cpu().numpy(), 1e-5, np.float32)
        tol = 2e-6 if odtype == torch.float32 else 2.0 ** -8
        np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize("M,N,K", [(1, 53, 29), (37, 64, 128), (130, 70, 33), (5, 311, 96)])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
def test_gemm_simt(M, N, K, adt, wdt):
    from gguf2bin_b200 import kernels
    a, w = rnd(M, K, dtype=adt, seed=3), rnd(N, K, dtype=wdt, seed=4)
    ref = a.double() @ w.double().T
    out = torch.empty(M, N, device=DEV)
    kernels.gemm_simt(a, w, out)
    assert (out.double() - ref).abs().max().item() < 1e-5 * math.sqrt(K) * 4
    base = rnd(M, N, seed=5)
    acc = base.clone()
    kernels.gemm_simt(a, w, acc, accumulate=True)
    assert (acc.double() - (base.double() + ref)).abs().max().item() < 1e-5 * math.sqrt(K) * 4
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.gemm_simt(a, w, out16)
    assert (out16.double() - ref).abs().max().item() <= (ref.abs().max().item() * 2.0 ** -8 + 1e-6)


def make_paged(n_seqs, lens, nkv, hd, page_size, dtype, seed):
    """Random K/V for sequences of the given lengths, scattered over shuffled pages.
    Returns (cache pages [n_pages,2,nkv,ps,hd], page_table [B,P], K list, V list)."""
    pages_per = [-(-l // page_size) for l in lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    cache = rnd(n_pages, 2, nkv, page_size, hd, dtype=dtype, seed=seed + 1)   # junk everywhere
    table = torch.zeros(n_seqs, max(pages_per), dtype=torch.int32)
    Ks, Vs, nxt = [], [], 0
    for b, l in enumerate(lens):
        K, V = rnd(l, nkv, hd, dtype=dtype, seed=seed + 10 + b), rnd(l, nkv, hd, dtype=dtype, seed=seed + 50 + b)
        for p in range(pages_per[b]):
            pg = perm[nxt]; nxt += 1
            table[b, p] = pg
            n = min(page_size, l - p * page_size)
            cache[pg, 0, :, :n] = K[p * page_size:p * page_size + n].transpose(0, 1)
            cache[pg, 1, :, :n] = V[p * page_size:p * page_size + n].transpose(0, 1)
        Ks.append(K); Vs.append(V)
    return cache, table.to(DEV), Ks, Vs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(6, 2, 48, 0), (4, 4, 16, 0), (5, 1, 80, 37), (8, 2, 128, 0)])
def test_attn_generic(dtype, nh, nkv, hd, window):
    """Ragged: sequence 0 a whole prompt, sequence 1 a prompt continued after a past,
    sequence 2 a single token far into its sequence."""
    from gguf2bin_b200 import kernels
    ps = 64
    lens = [70, 200, 333]
    q_lens = [70, 9, 1]
    cache, table, Ks, Vs = make_paged(3, lens, nkv, hd, ps, dtype, seed=7)
    tok_pos, tok_seq = [], []
    for b, (l, ql) in enumerate(zip(lens, q_lens)):
        tok_pos += list(range(l - ql, l)); tok_seq += [b] * ql
    T = len(tok_pos)
    q = rnd(T, nh * hd, dtype=dtype, seed=8)
    out = torch.empty_like(q)
    scale = 1 / math.sqrt(hd)
    kernels.attn_generic(q, out, cache, torch.tensor(tok_pos, dtype=torch.int32, device=DEV),
                         torch.tensor(tok_seq, dtype=torch.int32, device=DEV), table, nh, nkv, hd,
                         ps, window, scale)
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    t = 0
    for b, (l, ql) in enumerate(zip(lens, q_lens)):
        K, V = Ks[b].float().cpu().numpy(), Vs[b].float().cpu().numpy()
        qfull = np.zeros((l, nh, hd), np.float32)
        qfull[l - ql:] = q[t:t + ql].float().cpu().numpy().reshape(ql, nh, hd)
        ref = P.causal_attention(qfull, K, V, np.float32, window=window)[l - ql:]
        tol = 2e-5 if dtype == torch.float32 else 2.0 ** -7
        np.testing.assert_allclose(got[t:t + ql], ref, atol=tol * max(1, np.abs(ref).max()), rtol=0)
        t += ql


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,rot,norm", [(4, 2, 16, 16, True), (3, 1, 48, 32, True), (2, 2, 128, 128, False),
                                                (5, 1, 64, 64, True), (4, 2, 256, 256, True), (2, 1, 96, 96, True),
                                                (3, 3, 32, 32, True), (7, 1, 128, 128, True)])
@pytest.mark.parametrize("prompt", [70, 700])         # few rows: 4 elements per lane and half; many: 8
def test_qknorm_rope_cache(dtype, nh, nkv, hd, rot, norm, prompt):
    from gguf2bin_b200 import kernels
    ps, lens, q_lens = 64, [prompt, 130], [prompt, 2]
    cache, table, _, _ = make_paged(2, lens, nkv, hd, ps, dtype, seed=11)
    tok_pos, tok_seq = [], []
    for b, (l, ql) in enumerate(zip(lens, q_lens)):
        tok_pos += list(range(l - ql, l)); tok_seq += [b] * ql
    T = len(tok_pos)
    qkv = rnd(T, (nh + 2 * nkv) * hd, dtype=dtype, seed=12)
    qw, kw = (1 + 0.1 * rnd(hd, seed=13), 1 + 0.1 * rnd(hd, seed=14)) if norm else (None, None)
    theta, eps = 1e4, 1e-5
    inv_freq = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float().to(DEV)
    q_out = torch.empty(T, nh * hd, dtype=dtype, device=DEV)
    before = cache.clone()
    pos_t = torch.tensor(tok_pos, dtype=torch.int32, device=DEV)
    rope = torch.empty(T, rot // 2, 2, device=DEV)
    kernels.rope_table(pos_t, inv_freq, rope)
    kernels.qknorm_rope_cache(qkv, nh, nkv, hd, qw, kw, eps, rope, rot, pos_t,
                              torch.tensor(tok_seq, dtype=torch.int32, device=DEV), table, cache, ps, q_out)
    x = qkv.float().cpu().numpy().reshape(T, nh + 2 * nkv, hd)
    qq, kk, vv = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    if norm:
        qq = P.qk_rmsnorm(qq, qw.cpu().numpy(), eps, np.float32)
        kk = P.qk_rmsnorm(kk, kw.cpu().numpy(), eps, np.float32)

    def rope(a):
        r = P.rope_neox(a[..., :rot], tok_pos, theta, np.float32)
        return np.concatenate([r, a[..., rot:]], -1)
    qq, kk = rope(qq), rope(kk)
    tol = 3e-6 if dtype == torch.float32 else 2.0 ** -8
    np.testing.assert_allclose(q_out.float().cpu().numpy().reshape(T, nh, hd), qq, rtol=tol, atol=tol)
    touched = torch.zeros_like(cache, dtype=torch.bool)
    for t, (pos, b) in enumerate(zip(tok_pos, tok_seq)):
        pg = int(table[b, pos // ps])
        np.testing.assert_allclose(cache[pg, 0, :, pos % ps].float().cpu().numpy(), kk[t], rtol=tol, atol=tol)
        np.testing.assert_allclose(cache[pg, 1, :, pos % ps].float().cpu().numpy(), vv[t], rtol=tol, atol=tol)
        touched[pg, :, :, pos % ps] = True
    assert torch.equal(cache[~touched], before[~touched]), "cache written outside the tokens' places"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I,blk", [(24, 8), (100, 100), (224, 8)])
def test_swiglu(dtype, I, blk):
    from gguf2bin_b200 import kernels
    T = 5
    g, u = rnd(T, I, dtype=dtype, seed=20), rnd(T, I, dtype=dtype, seed=21)
    fused = torch.stack([g.view(T, I // blk, blk), u.view(T, I // blk, blk)], dim=2).reshape(T, 2 * I).contiguous()
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    kernels.swiglu(fused, out, blk)
    gf, uf = g.float(), u.float()
    ref = (gf / (1 + torch.exp(-gf))) * uf
    tol = 1e-6 if dtype == torch.float32 else 2.0 ** -8
    assert ((out.float() - ref).abs() <= tol * (1 + ref.abs())).all()


def test_sampling_greedy_and_temperature():
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS
    R, V = 6, 1537
    logits = rnd(R, V, scale=3.0, seed=30)
    logits[0, 100] = logits[0, 900] = 50.0            # a tie: the lower id wins
    state = torch.zeros(8, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.tensor([3, 1, 4, 0, 5, 7], dtype=torch.int32, device=DEV)
    streams = torch.tensor([10, 11, 12, 13, 14, 15], dtype=torch.int32, device=DEV)
    seed = 0x1234567890ABCDEF
    kernels.seed_slots(state, slots, streams, seed)
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    kernels.sample_rows(logits, 0.0, state, slots, ids)
    assert ids.tolist() == [P.greedy(l) for l in logits.cpu().numpy()]
    assert ids[0].item() == 100
    for draw in range(3):
        kernels.sample_rows(logits, 0.8, state, slots, ids)
        for r in range(R):
            u = philox_plain.uniform(seed, 10 + r, draw)
            want, cdf = P.sample_temperature(logits[r].cpu().numpy(), 0.8, u)
            got = ids[r].item()
            lo = cdf[got - 1] if got > 0 else 0.0
            assert lo - 1e-5 <= u <= cdf[got] + 1e-5, (r, draw, got, want, u)
    assert state[slots.long(), 3].tolist() == [3] * R


@pytest.mark.parametrize("V,scale", [(151936, 3.0), (8192, 0.5), (300001, 6.0), (40003, 30.0)])
def test_temperature_sampling_of_a_large_vocabulary(V, scale):
    """From 8,192 entries on, many blocks per row sum the row's pieces (each against its own
    maximum) before the row's block draws: a vocabulary of the real size, the smallest that takes
    this way, one whose pieces are 256 entries, one that is no multiple of four (unaligned rows);
    flat and peaked rows; a row whose maximum is in its last, partial piece."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS
    R = 5
    logits = rnd(R, V, scale=scale, seed=33)
    logits[1, V - 1] = logits[1].max() + 4.0
    logits[2, 7] = logits[2].max() + 9.0              # most of the mass in one entry
    state = torch.zeros(R, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.tensor([2, 0, 4, 1, 3], dtype=torch.int32, device=DEV)
    seed = 4321
    kernels.seed_slots(state, slots, torch.arange(R, dtype=torch.int32, device=DEV), seed)
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    # The cumulative distribution of src/l5_model.c:615-619 with the sums taken in float64: the plain
    # sampler adds 150k float32 terms one after the other, as the reference does, and its total is
    # off by 2.5e-4 at this size, which is no property to reproduce.
    cdfs = []
    for row in logits.cpu().numpy():
        x = (row / np.float32(0.9)).astype(np.float64)
        e = np.exp(x - x.max())
        cdfs.append(np.cumsum(e) / e.sum())
    chosen = set()
    for draw in range(6):
        kernels.sample_rows(logits, 0.9, state, slots, ids)
        for r in range(R):
            u = philox_plain.uniform(seed, r, draw)
            got = ids[r].item()
            lo = cdfs[r][got - 1] if got > 0 else 0.0
            assert lo - 1e-5 <= u <= cdfs[r][got] + 1e-5, (r, draw, got, u)
            chosen.add(got)
    assert scale > 10 or len(chosen) > R


@pytest.mark.parametrize("V,ties", [(2011, False), (151936, False), (40000, True)])
@pytest.mark.parametrize("top_k,top_p,penalty", [(40, 0.9, 1.1), (0, 0.9, 1.0), (5, 1.0, 1.3), (0, 1.0, 1.0), (1, 0.5, 1.0),
                                                 (2048, 0.95, 1.0), (3000, 0.9, 1.1), (64, 0.99, 1.1), (100, 0.9, 1.1),
                                                 (256, 1.0, 1.0), (257, 0.97, 1.2)])
def test_sampling_filtered(top_k, top_p, penalty, V, ties):
    """Repeat penalty, top-k, top-p and the draw against the plain sampler: a small and a real
    vocabulary; a top_k that is listed and sorted (up to 2,048) and one that is not; and logits
    rounded to tenths, so that hundreds of entries tie at every cut and the listed path gives
    way to the descents over the whole row."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS
    R, temp = 5, 0.7
    logits = rnd(R, V, scale=2.5, seed=31)
    if ties:
        logits = (logits * 10).round() / 10
    recent = torch.randint(0, V, (R, 64), generator=torch.Generator().manual_seed(5), dtype=torch.int32)
    recent[:, 10] = recent[:, 3]                       # a repeated id is penalised once
    recent_n = torch.tensor([64, 0, 17, 64, 1], dtype=torch.int32)
    state = torch.zeros(R, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.arange(R, dtype=torch.int32, device=DEV)
    seed = 77
    kernels.seed_slots(state, slots, slots.clone(), seed)
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    for draw in range(4):
        work = logits.clone()
        kernels.sample_filtered(work, temp, top_k, top_p, penalty, recent.to(DEV), recent_n.to(DEV),
                                state, slots, ids)
        for r in range(R):
            u = philox_plain.uniform(seed, r, draw)
            rec = recent[r, :recent_n[r]].tolist()
            want, kept, cdf = P.sample_advanced(logits[r].cpu().numpy(), temp, top_k, top_p, penalty, rec, u)
            got = ids[r].item()
            where = np.nonzero(kept == got)[0]
            assert len(where) == 1, (r, draw, got, "not in the kept set", len(kept))
            i = int(where[0])
            lo = cdf[i - 1] if i > 0 else 0.0
            assert lo - 1e-4 <= u <= cdf[i] + 1e-4, (r, draw, got, want, u, lo, cdf[i])
    # greedy through the same kernel applies the penalty first
    work = logits.clone()
    kernels.sample_filtered(work, 0.0, top_k, top_p, penalty, recent.to(DEV), recent_n.to(DEV), state, slots, ids)
    for r in range(R):
        rec = recent[r, :recent_n[r]].tolist()
        assert ids[r].item() == P.sample_advanced(logits[r].cpu().numpy(), 0.0, top_k, top_p, penalty, rec, 0.5)[0]


@pytest.mark.parametrize("V,scale,top_p,penalty", [(151936, 2.5, 0.9, 1.0), (151936, 2.5, 1.0, 1.2), (151936, 12.0, 0.95, 1.1),
                                                   (50021, 0.3, 0.5, 1.0), (9001, 40.0, 0.9, 1.0), (300, 2.0, 0.8, 1.3)])
def test_sampling_without_a_top_k(V, scale, top_p, penalty):
    """No top_k: a top_p alone, or only the repeat penalty.  Flat rows, of which the top_p keeps tens
    of thousands of entries, and peaked ones, of which it keeps one or two; a row whose values all lie
    within a few buckets; every draw against the plain sampler's kept set and cumulative sums."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS
    R, temp = 4, 0.7
    logits = rnd(R, V, scale=scale, seed=36)
    recent = torch.randint(0, V, (R, 64), generator=torch.Generator().manual_seed(7), dtype=torch.int32)
    recent[:, :4] = logits.topk(4, dim=1).indices.cpu().to(torch.int32)
    recent_n = torch.tensor([64, 0, 30, 64], dtype=torch.int32)
    state = torch.zeros(R, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.arange(R, dtype=torch.int32, device=DEV)
    seed = 79
    kernels.seed_slots(state, slots, slots.clone(), seed)
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    host = logits.cpu().numpy()
    sizes = set()
    for draw in range(5):
        work = logits.clone()
        kernels.sample_filtered(work, temp, 0, top_p, penalty, recent.to(DEV), recent_n.to(DEV), state, slots, ids)
        for r in range(R):
            u = philox_plain.uniform(seed, r, draw)
            want, kept, cdf = P.sample_advanced(host[r], temp, 0, top_p, penalty, recent[r, :recent_n[r]].tolist(), u)
            got = ids[r].item()
            where = np.nonzero(kept == got)[0]
            assert len(where) == 1, (r, draw, got, "not in the kept set", len(kept))
            i = int(where[0])
            lo = cdf[i - 1] if i > 0 else 0.0
            assert lo - 1e-4 <= u <= cdf[i] + 1e-4, (r, draw, got, want, u, lo, cdf[i])
            sizes.add(len(kept))
    assert state[:, 3].tolist() == [5] * R, "one random number per token"
    assert scale > 10 or V < 1000 or max(sizes) > 100


@pytest.mark.parametrize("R", [40, 100, 160])
def test_sampling_filtered_many_rows(R):
    """With many rows the rows are cut into fewer slices (16, 8, 4; none beyond what fills the GPU
    once): every row against the plain sampler, with ids of the penalty in every slice."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS
    V, temp, top_k, top_p, penalty = 151936, 0.7, 40, 0.9, 1.3
    logits = rnd(R, V, scale=2.5, seed=35)
    g = torch.Generator().manual_seed(6)
    recent = torch.randint(0, V, (R, 64), generator=g, dtype=torch.int32)
    top = logits.topk(8, dim=1).indices.cpu().to(torch.int32)
    recent[:, :8] = top                                # the penalty reorders the head of every row
    recent_n = torch.full((R,), 64, dtype=torch.int32)
    state = torch.zeros(R, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.arange(R, dtype=torch.int32, device=DEV)
    seed = 78
    kernels.seed_slots(state, slots, slots.clone(), seed)
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    work = logits.clone()
    kernels.sample_filtered(work, temp, top_k, top_p, penalty, recent.to(DEV), recent_n.to(DEV), state, slots, ids)
    host = logits.cpu().numpy()
    for r in range(R):
        u = philox_plain.uniform(seed, r, 0)
        want, kept, cdf = P.sample_advanced(host[r], temp, top_k, top_p, penalty, recent[r].tolist(), u)
        got = ids[r].item()
        where = np.nonzero(kept == got)[0]
        assert len(where) == 1, (r, got, "not in the kept set", len(kept))
        i = int(where[0])
        lo = cdf[i - 1] if i > 0 else 0.0
        assert lo - 1e-4 <= u <= cdf[i] + 1e-4, (r, got, want, u, lo, cdf[i])


def test_sampling_with_the_recent_ids_on_the_device():
    """The repeat penalty over the ids in the sequences' own records: started with a prompt's
    tail (three, sixty-four and no ids), extended by every sampled id, across the ring's wrap,
    and with one step taken back; every draw against the plain sampler given the same window."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.cache import SEQ_STATE_WORDS, SS_RECENT_TOTAL
    R, V, temp, top_k, top_p, penalty = 3, 1009, 0.7, 20, 0.9, 1.5
    seed = 99
    state = torch.zeros(5, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
    slots = torch.tensor([4, 0, 2], dtype=torch.int32, device=DEV)
    kernels.seed_slots(state, slots, torch.arange(R, dtype=torch.int32, device=DEV), seed)
    g = torch.Generator().manual_seed(3)
    windows = [torch.randint(0, V, (n,), generator=g).tolist() for n in (3, 64, 0)]
    rows = torch.zeros(R, 65, dtype=torch.int32)
    for r, w in enumerate(windows):
        rows[r, 0] = len(w)
        rows[r, 1:1 + len(w)] = torch.tensor(w, dtype=torch.int32)
    kernels.recent_set(state, slots, rows.to(DEV))
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    draws = [0] * R
    for step in range(90):                               # past the ring's 72 places
        logits = rnd(R, V, scale=2.5, seed=400 + step)
        work = logits.clone()
        kernels.sample_filtered(work, temp, top_k, top_p, penalty, None, None, state, slots, ids, append=True)
        got = ids.tolist()
        for r in range(R):
            u = philox_plain.uniform(seed, r, draws[r])
            _, kept, cdf = P.sample_advanced(logits[r].cpu().numpy(), temp, top_k, top_p, penalty, windows[r][-64:], u)
            where = np.nonzero(kept == got[r])[0]
            assert len(where) == 1, (step, r, got[r], "not in the kept set")
            i = int(where[0])
            assert (cdf[i - 1] if i > 0 else 0.0) - 1e-4 <= u <= cdf[i] + 1e-4, (step, r)
            draws[r] += 1
            windows[r].append(got[r])
        if step % 7 == 3:                                # this step is taken back: its id and its draw do not count
            pos = torch.zeros(R, dtype=torch.int32, device=DEV)
            kernels.rewind_step(pos, R, state, slots, True, True)
            for r in range(R):
                windows[r].pop()
                draws[r] -= 1
    assert state[slots.long(), SS_RECENT_TOTAL].tolist() == [len(w) for w in windows]


@pytest.mark.parametrize("fine", [False, True])
@pytest.mark.parametrize("nh,nkv,hd,window", [(16, 8, 128, 0), (5, 1, 128, 0), (20, 1, 64, 0), (6, 2, 64, 300),
                                              (4, 4, 128, 70)])
def test_attn_decode(nh, nkv, hd, window, fine):
    """Split-key decode attention: one token per sequence at positions before, at and
    after chunk (256, or 128 with ``fine``) and page (64) edges; groups of 1, 2, 5 and 20 query heads per kv
    head; a window that starts inside a chunk."""
    from types import SimpleNamespace
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.engine.workspace import Workspace
    ps = 64
    lens = [1, 63, 64, 65, 255, 256, 257, 700, 1025]
    cache, table, Ks, Vs = make_paged(len(lens), lens, nkv, hd, ps, torch.bfloat16, seed=40)
    T = len(lens)
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=41)
    # make one far key stand out for the longest sequence
    Ks[-1][17] = (q[-1].view(nh, hd)[0] * 0.5)[None, :].expand(nkv, hd)
    pg = int(table[T - 1, 0])
    cache[pg, 0, :, 17] = Ks[-1][17]
    out = torch.empty_like(q)
    ctx = SimpleNamespace(tok_pos=torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV),
                          tok_seq=torch.arange(T, dtype=torch.int32, device=DEV), page_table=table,
                          max_kv_len=table.shape[1] * ps, workspace=Workspace(DEV), all_single=True)
    scale = 1 / math.sqrt(hd)
    kernels_bf16.attn_decode(q, out, cache, ctx, nh, nkv, hd, ps, window, scale, fine=fine)
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    for b, l in enumerate(lens):
        K, V = Ks[b].float().cpu().numpy(), Vs[b].float().cpu().numpy()
        qfull = np.zeros((l, nh, hd), np.float32)
        qfull[-1] = q[b].float().cpu().numpy().reshape(nh, hd)
        ref = P.causal_attention(qfull, K, V, np.float32, window=window)[-1]
        np.testing.assert_allclose(got[b], ref, atol=2.0 ** -7 * max(1, np.abs(ref).max()), rtol=0,
                                   err_msg=f"sequence of {l} keys")


@pytest.mark.parametrize("M,N,K", [(1, 4096, 1024), (8, 6144, 1024), (13, 1008, 520), (16, 2048 + 16, 1280),
                                   (5, 311 * 16, 72), (3, 48, 2056)])
def test_normed_product(M, N, K):
    """The few-row product that normalises its own rows: norm(x) . W^T with the row's
    1 / sqrt(mean(x^2) + eps) applied to the accumulators, plain and with the SiLU gate,
    against float64; rows of very different size (the factor is per row)."""
    from gguf2bin_b200 import kernels, kernels_bf16
    x = rnd(M, K, seed=70) * torch.logspace(-2, 2, M, device=DEV)[:, None]
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=71)
    eps = 1e-5
    xb = x.to(torch.bfloat16).double()                                  # what the tensor cores are fed
    inv = 1 / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps)
    ref = (xb @ w.double().T) * inv
    tol = 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item())
    out = torch.full((M, N), 7.0, device=DEV)
    assert kernels.normed_product(x, eps, w, out)
    assert (out.double() - ref).abs().max().item() < tol
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert kernels.normed_product(x, eps, w, out16)
    assert (out16.double() - ref).abs().max().item() <= ref.abs().max().item() * 2.0 ** -8 + tol
    I = N // 2
    g = ref.view(M, I // 8, 2, 8)[:, :, 0].reshape(M, I)
    u = ref.view(M, I // 8, 2, 8)[:, :, 1].reshape(M, I)
    want = (g / (1 + torch.exp(-g))) * u
    mid = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    assert kernels.normed_product(x, eps, w, mid, gate_block=8)
    assert (mid.double() - want).abs().max().item() <= want.abs().max().item() * 2.0 ** -8 + tol
    # and it is the norm kernel without a weight followed by the product, up to the rounding of the normed rows
    h = torch.empty(M, K, dtype=torch.bfloat16, device=DEV)
    kernels.rmsnorm(x, None, eps, h)
    two = torch.empty(M, N, device=DEV)
    kernels.linear(h, w, two)
    assert (two.double() - ref).abs().max().item() <= 2.0 ** -7 * ref.abs().max().item() + tol
    # cases that are left to the two kernels
    assert not kernels.normed_product(rnd(17, K, seed=1), eps, w, torch.empty(17, N, device=DEV))
    assert not kernels.normed_product(rnd(4, 4096, seed=1), eps, rnd(1024, 4096, dtype=torch.bfloat16), torch.empty(4, 1024, device=DEV))


def last_row_attention(q_row, K, V, nh, window):
    """The last token's row of ``P.causal_attention`` (same formula: src/l5_model.c:518, 559-577,
    softmax src/l3_math.c:52-56), computed alone so that thousands of keys stay quick."""
    l, nkv, hd = K.shape
    group, lo = nh // nkv, (0 if window <= 0 else max(0, l - window))
    out = np.zeros((nh, hd), np.float32)
    for h in range(nh):
        s = (K[lo:, h // group] @ q_row[h]) * (np.float32(1) / np.sqrt(np.float32(hd)))
        e = np.exp(s - s.max())
        out[h] = (e / e.sum(dtype=np.float32)) @ V[lo:, h // group]
    return out


@pytest.mark.parametrize("fine", [False, True])
@pytest.mark.parametrize("nh,nkv,hd,window", [(16, 8, 128, 0), (8, 2, 64, 0), (16, 8, 128, 3000)])
def test_attn_decode_long_and_wide(nh, nkv, hd, window, fine):
    """Twenty sequences of up to 4,100 keys (17 chunks of 256, 33 of 128): the merge of many
    chunks by four warps, chunk counts that are and are not multiples of four, a window that
    drops whole chunks.  A planted key far back takes most of one sequence's attention."""
    from types import SimpleNamespace
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.engine.workspace import Workspace
    ps = 64
    lens = [4100, 4096, 4095, 3073, 2049, 2048, 1500, 1281, 1024, 1023, 777, 513, 512, 300, 129, 64, 17, 1, 3584, 2817]
    cache, table, Ks, Vs = make_paged(len(lens), lens, nkv, hd, ps, torch.bfloat16, seed=140)
    T = len(lens)
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=141)
    Ks[0][1300] = (q[0].view(nh, hd)[0] * 0.5)[None, :].expand(nkv, hd)       # in chunk 5 of 17
    cache[int(table[0, 1300 // ps]), 0, :, 1300 % ps] = Ks[0][1300]
    out = torch.empty_like(q)
    ctx = SimpleNamespace(tok_pos=torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV),
                          tok_seq=torch.arange(T, dtype=torch.int32, device=DEV), page_table=table,
                          max_kv_len=table.shape[1] * ps, workspace=Workspace(DEV), all_single=True)
    kernels_bf16.attn_decode(q, out, cache, ctx, nh, nkv, hd, ps, window, 1 / math.sqrt(hd), fine=fine)
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    for b, l in enumerate(lens):
        ref = last_row_attention(q[b].float().cpu().numpy().reshape(nh, hd), Ks[b].float().cpu().numpy(),
                                 Vs[b].float().cpu().numpy(), nh, window)
        np.testing.assert_allclose(got[b], ref, atol=2.0 ** -7 * max(1, np.abs(ref).max()), rtol=0,
                                   err_msg=f"sequence of {l} keys")
    small = last_row_attention(q[0].float().cpu().numpy().reshape(nh, hd), Ks[0].float().cpu().numpy()[:300],
                               Vs[0].float().cpu().numpy()[:300], nh, 0)
    assert window or np.abs(got[0][0] - Vs[0][1300, 0].float().cpu().numpy()).max() < \
        np.abs(small[0] - Vs[0][1300, 0].float().cpu().numpy()).max(), "the planted key does not stand out"


@pytest.mark.parametrize("M,N,K", [(1, 48, 64), (8, 1024, 2048), (3, 200, 264), (16, 96, 1032),
                                   (33, 1000, 520), (64, 311, 96),
                                   # many tiles per CTA: groups of 1, 2, 4, 8 tiles, one and several chunks of K,
                                   # a last chunk and a last group that are not full, 8 and 16 staged rows
                                   (1, 4096, 4096), (8, 6144, 4096), (5, 2400 + 8, 2056), (16, 5120, 3080),
                                   (3, 40000, 2048), (11, 24576, 2048), (7, 80000 + 24, 2304)])
def test_gemm_small(M, N, K):
    """Weight-streaming product for few rows: every epilogue, widths that are no multiple
    of the 16-row tile or of the 256-wide K block."""
    from gguf2bin_b200 import kernels_bf16
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=60), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=61)
    ref = a.double() @ w.double().T
    tol = 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item())
    out = torch.full((M, N), 7.0, device=DEV)
    assert kernels_bf16.linear_bf16(a, w, out, False)
    assert (out.double() - ref).abs().max().item() < tol
    base = rnd(M, N, seed=62)
    acc = base.clone()
    assert kernels_bf16.linear_bf16(a, w, acc, True)
    assert (acc.double() - base.double() - ref).abs().max().item() < tol
    out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    assert kernels_bf16.linear_bf16(a, w, out16, False)
    assert (out16.double() - ref).abs().max().item() <= ref.abs().max().item() * 2.0 ** -8 + tol
    # a row changes nothing in the other rows: bit-equal when run alone (by the same family of kernels)
    if M > 1 and kernels_bf16._pick_product(a, w) == "small":
        alone = torch.empty(1, N, device=DEV)
        kernels_bf16.linear_bf16(a[M - 1:M], w, alone, False)
        assert torch.equal(alone[0], out[M - 1])
    if N % 16 == 0:
        I = N // 2
        g = ref.view(M, I // 8, 2, 8)[:, :, 0].reshape(M, I)
        u = ref.view(M, I // 8, 2, 8)[:, :, 1].reshape(M, I)
        want = (g / (1 + torch.exp(-g))) * u
        mid = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        assert kernels_bf16.gate_up_bf16(a, w, mid, 8)
        assert (mid.double() - want).abs().max().item() <= want.abs().max().item() * 2.0 ** -8 + tol


@pytest.mark.parametrize("kernel", ["mma", "tcgen05", "tcgen05 split"])
@pytest.mark.parametrize("nh,nkv,hd,window", [(16, 8, 128, 0), (5, 1, 128, 0), (6, 2, 64, 0), (4, 2, 64, 100),
                                              (2, 2, 128, 33)])
def test_attn_prefill(nh, nkv, hd, window, kernel):
    """Prompt attention: a whole prompt that is no multiple of the 64-row tile, a prompt
    continued after a past that ends inside a page, a single token far into a sequence,
    and a short prompt; windows that start inside a page."""
    from types import SimpleNamespace
    from gguf2bin_b200 import kernels_bf16
    ps = 64
    lens = [333, 200, 700, 5]
    q_lens = [333, 70, 1, 5]
    cache, table, Ks, Vs = make_paged(len(lens), lens, nkv, hd, ps, torch.bfloat16, seed=70)
    rows = 64 if kernel == "mma" else 128
    tiles, t0 = [], 0
    for b, (l, ql) in enumerate(zip(lens, q_lens)):
        for r in range(0, ql, rows):
            tiles.append((b, t0 + r, min(rows, ql - r), l - ql + r))
        t0 += ql
    T = t0
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=71)
    out = torch.zeros_like(q)
    tt = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    if kernel == "mma":
        ctx = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles=len(tiles), attn_tiles=tt)
        kernels_bf16.attn_prefill(q, out, cache, ctx, nh, nkv, hd, ps, window, 1 / math.sqrt(hd))
    else:
        ctx = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles_wide=len(tiles), attn_tiles_wide=tt)
        kernels_bf16.attn_prefill_tc(q, out, cache, ctx, nh, nkv, hd, ps, window, 1 / math.sqrt(hd),
                                     split=kernel.endswith("split"))
        kernels_bf16.check_status()
    got = out.float().cpu().numpy().reshape(T, nh, hd)
    t = 0
    for b, (l, ql) in enumerate(zip(lens, q_lens)):
        K, V = Ks[b].float().cpu().numpy(), Vs[b].float().cpu().numpy()
        qfull = np.zeros((l, nh, hd), np.float32)
        qfull[l - ql:] = q[t:t + ql].float().cpu().numpy().reshape(ql, nh, hd)
        ref = P.causal_attention(qfull, K, V, np.float32, window=window)[l - ql:]
        np.testing.assert_allclose(got[t:t + ql], ref, atol=2.0 ** -7 * max(1, np.abs(ref).max()), rtol=0,
                                   err_msg=f"sequence {b}")
        t += ql


def row_attention(q_row, K, V, nh, pos, window=0):
    """Row ``pos`` of the plain causal attention (keys 0..pos, or the last ``window`` of them)."""
    lo = 0 if window <= 0 else max(0, pos - window + 1)
    return last_row_attention(q_row, K[:pos + 1], V[:pos + 1], nh, pos + 1 - lo if window > 0 else 0)


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("window", [0, 5000])
def test_attention_over_tens_of_thousands_of_keys(window, split):
    """A prompt of 20,000 tokens (157 query tiles, up to 313 pages per tile) through the tcgen05
    prompt attention (both kernels), then one token at position 39,999 of a sequence of 40,000 through the
    decode attention: rows at the start, at tile and page edges, in the middle and at the end
    against the plain attention of that row; a planted key 19,000 positions back stands out."""
    from types import SimpleNamespace
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.engine.workspace import Workspace
    nh, nkv, hd, ps = 4, 2, 128, 64
    lens = [20000, 40000]
    cache, table, Ks, Vs = make_paged(2, lens, nkv, hd, ps, torch.bfloat16, seed=170)
    scale = 1 / math.sqrt(hd)
    # sequence 0: the whole prompt
    T = lens[0]
    q = rnd(T, nh * hd, dtype=torch.bfloat16, seed=171)
    Ks[0][700] = (q[19700].view(nh, hd)[0] * 0.5)[None, :].expand(nkv, hd)      # row 19,700 looks 19,000 back
    cache[int(table[0, 700 // ps]), 0, :, 700 % ps] = Ks[0][700]
    tiles = sorted([(0, r, min(128, T - r), r) for r in range(0, T, 128)], key=lambda t: -t[3])
    ctx = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles_wide=len(tiles),
                          attn_tiles_wide=torch.tensor(tiles, dtype=torch.int32, device=DEV))
    out = torch.zeros_like(q)
    kernels_bf16.attn_prefill_tc(q, out, cache, ctx, nh, nkv, hd, ps, window, scale, split=split)
    kernels_bf16.check_status()
    K, V = Ks[0].float().cpu().numpy(), Vs[0].float().cpu().numpy()
    for pos in (0, 63, 64, 127, 128, 9999, 16383, 16384, 19700, 19999):
        ref = row_attention(q[pos].float().cpu().numpy().reshape(nh, hd), K, V, nh, pos, window)
        got = out[pos].float().cpu().numpy().reshape(nh, hd)
        np.testing.assert_allclose(got, ref, atol=2.0 ** -7 * max(1, np.abs(ref).max()), rtol=0, err_msg=f"row {pos}")
    if not window:
        far = np.abs(out[19700].float().cpu().numpy().reshape(nh, hd)[0] - Vs[0][700, 0].float().cpu().numpy()).max()
        near = np.abs(out[19699].float().cpu().numpy().reshape(nh, hd)[0] - Vs[0][700, 0].float().cpu().numpy()).max()
        assert far < near, "the planted key does not stand out"
    # sequence 1: one token at the end of 40,000 keys
    q1 = rnd(1, nh * hd, dtype=torch.bfloat16, seed=172)
    out1 = torch.zeros_like(q1)
    dctx = SimpleNamespace(tok_pos=torch.tensor([lens[1] - 1], dtype=torch.int32, device=DEV),
                           tok_seq=torch.tensor([1], dtype=torch.int32, device=DEV), page_table=table,
                           max_kv_len=table.shape[1] * ps, workspace=Workspace(DEV), all_single=True)
    kernels_bf16.attn_decode(q1, out1, cache, dctx, nh, nkv, hd, ps, window, scale)
    ref = row_attention(q1[0].float().cpu().numpy().reshape(nh, hd), Ks[1].float().cpu().numpy(),
                        Vs[1].float().cpu().numpy(), nh, lens[1] - 1, window)
    np.testing.assert_allclose(out1.float().cpu().numpy().reshape(nh, hd), ref,
                               atol=2.0 ** -7 * max(1, np.abs(ref).max()), rtol=0, err_msg="decode at 40,000 keys")


def _check_gemm_tc_epilogue(M, N, K, bn, stages, persistent, epi):
    """One epilogue of the tcgen05 product against float64."""
    from gguf2bin_b200 import kernels_bf16
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=80), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=81)
    ref = a.double() @ w.double().T
    tol = 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item())
    if epi == kernels_bf16.EPI_STORE_F32:
        out = torch.full((M, N), 7.0, device=DEV)
        kernels_bf16._gemm_tc(a, w, out, epi, bn, stages, persistent)
        kernels_bf16.check_status()
        assert (out.double() - ref).abs().max().item() < tol
    elif epi == kernels_bf16.EPI_ACCUM_F32:
        base = rnd(M, N, seed=82)
        acc = base.clone()
        kernels_bf16._gemm_tc(a, w, acc, epi, bn, stages, persistent)
        assert (acc.double() - base.double() - ref).abs().max().item() < tol
    elif epi == kernels_bf16.EPI_STORE_BF16:
        out16 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        kernels_bf16._gemm_tc(a, w, out16, epi, bn, stages, persistent)
        assert (out16.double() - ref).abs().max().item() <= ref.abs().max().item() * 2.0 ** -8 + tol
    else:
        I = N // 2
        g = ref.view(M, I // 8, 2, 8)[:, :, 0].reshape(M, I)
        u = ref.view(M, I // 8, 2, 8)[:, :, 1].reshape(M, I)
        want = (g / (1 + torch.exp(-g))) * u
        mid = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
        kernels_bf16._gemm_tc(a, w, mid, epi, bn, stages, persistent)
        assert (mid.double() - want).abs().max().item() <= want.abs().max().item() * 2.0 ** -8 + tol
    kernels_bf16.check_status()


def _check_gemm_tc(M, N, K, bn, stages, persistent):
    from gguf2bin_b200 import kernels_bf16
    for epi in (kernels_bf16.EPI_STORE_F32, kernels_bf16.EPI_ACCUM_F32, kernels_bf16.EPI_STORE_BF16):
        _check_gemm_tc_epilogue(M, N, K, bn, stages, persistent, epi)
    if N % 16 == 0:
        _check_gemm_tc_epilogue(M, N, K, bn, stages, persistent, kernels_bf16.EPI_SWIGLU_BF16)


@pytest.mark.parametrize("bn,stages", [(64, 4), (64, 8), (128, 3), (128, 6), (256, 4), (0, 0)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (65, 256, 128), (200, 1000, 1032), (333, 96, 96),
                                   (1024, 512, 2048), (129, 311 * 8, 72)])
def test_gemm_tc(M, N, K, bn, stages):
    """tcgen05 product: one and many K blocks, ragged M / N / K tails, every epilogue."""
    _check_gemm_tc(M, N, K, bn, stages, False)


@pytest.mark.parametrize("bn,stages", [(128, 6), (256, 4)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 1000, 1032), (2048 + 17, 2560 + 8, 320),
                                   (4096, 2048, 136), (1500, 6144, 1024)])
def test_gemm_tc_persistent(M, N, K, bn, stages):
    """The persistent variant: fewer tiles than SMs, and several tiles per CTA (both
    accumulators in use, the ring running across tile borders), ragged tails, every epilogue."""
    _check_gemm_tc(M, N, K, bn, stages, True)


@pytest.mark.parametrize("M,N,K", [(300, 528, 1096), (129, 256, 2048), (1000, 1008, 4096), (640, 2048, 1024),
                                   (2048, 1024, 3072), (256, 1024, 3072 + 8)])
def test_gemm_tc_persistent_k_in_parts(M, N, K):
    """Few tiles: the persistent kernel takes K in 2, 3 or 4 parts over a cluster, whose ranks
    exchange their partial tiles through the cluster's shared memory and add them in rank order.
    Every epilogue and both tile widths, by hand and as the launcher chooses (width 0); a number
    of parts that the tile, the epilogue or the GPU cannot take is refused, never computed wrongly;
    the same bits on every run."""
    from gguf2bin_b200 import kernels_bf16
    from gguf2bin_b200.kernels import KernelError
    ran = {}
    for bn, stages in ((128, 6), (256, 4)):
        for parts in (2, 3, 4):
            for epi in (kernels_bf16.EPI_ACCUM_F32, kernels_bf16.EPI_STORE_F32, kernels_bf16.EPI_STORE_BF16,
                        kernels_bf16.EPI_SWIGLU_BF16):
                try:
                    _check_gemm_tc_epilogue(M, N, K, bn, stages, 10 + parts, epi)
                    ran[epi] = ran.get(epi, 0) + 1
                except KernelError as e:
                    assert "parts of K" in str(e), str(e)
            a, w = rnd(M, K, dtype=torch.bfloat16, seed=80), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=81)
            outs = []
            try:
                for _ in range(3):
                    out = torch.ones(M, N, device=DEV)
                    kernels_bf16._gemm_tc(a, w, out, kernels_bf16.EPI_ACCUM_F32, bn, stages, 10 + parts)
                    outs.append(out)
            except KernelError:
                continue
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), (bn, parts)
    assert all(ran.get(epi, 0) >= 1 for epi in (0, 1, 2, 3)), ran
    _check_gemm_tc(M, N, K, 0, 0, True)
    _check_gemm_tc(M, N, K, 128, 6, True)
    _check_gemm_tc(M, N, K, 256, 4, True)


@pytest.mark.parametrize("bn,stages", [(256, 6), (256, 4)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (200, 1000, 1032), (2048 + 17, 2560 + 8, 320),
                                   (4096, 2048, 136), (1500, 6144, 1024), (129, 130 * 8, 72),
                                   # a long K at a thousand rows: where prompts against big weights take this kernel
                                   (1100, 4096, 4096), (1024, 2048 + 16, 12288 + 8)])
def test_gemm_tc_pairs(M, N, K, bn, stages):
    """The product on pairs of CTAs (cta_group::2, tiles of 256 rows): one tile and several per
    pair, a peer CTA whose rows of A or of W lie wholly or partly outside, every epilogue."""
    _check_gemm_tc(M, N, K, bn, stages, 2)


@pytest.mark.parametrize("M,N,K", [(9, 4096, 2048), (17, 4096, 4096), (32, 2048 + 8, 2048), (33, 6144, 4096), (64, 4096, 12288),
                                   (100, 2304, 2056), (128, 4096 + 24, 4096 + 8), (20, 130 * 8, 72),
                                   (64, 5120, 5120), (23, 5120 + 8, 1096)])
def test_gemm_tc_weight_streaming(M, N, K):
    """17 to 128 rows against big weights: 128 rows of W per CTA with 32, 64 or 128 rows of A,
    K in 1, 2, 3 and 4 parts added in rank order through the cluster's shared memory (three
    where four would not fit the GPU at once: 40 and 48 tiles), ragged N and K, every epilogue;
    the same bits on every run; and every number of parts asked for by hand."""
    from gguf2bin_b200 import kernels_bf16
    _check_gemm_tc(M, N, K, 0, 0, 3)
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=80), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=81)
    outs = []
    for _ in range(3):
        out = torch.zeros(M, N, device=DEV)
        kernels_bf16._gemm_tc(a, w, out, kernels_bf16.EPI_ACCUM_F32, 0, 0, 3)
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ref = a.double() @ w.double().T
    for parts in (1, 2, 3, 4):
        out = torch.zeros(M, N, device=DEV)
        kernels_bf16._gemm_tc(a, w, out, kernels_bf16.EPI_STORE_F32, parts, 0, 3)
        assert (out.double() - ref).abs().max().item() < 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item()), parts
    kernels_bf16.check_status()


@pytest.mark.parametrize("mode,bn,stages", [(True, 256, 4), (2, 256, 6)])
def test_gemm_tc_rows_in_groups(mode, bn, stages):
    """An A operand larger than the L2 makes the persistent kernels walk the rows of tiles in
    groups (here two groups, the second shorter, three columns of tiles): every tile still once."""
    _check_gemm_tc(8192 + 40, 520, 4104, bn, stages, mode)


def test_linear_of_a_long_prompt_runs_on_pairs():
    """From 4,096 rows on the product is given to pairs of CTAs; the same result as the plain one."""
    from gguf2bin_b200 import kernels_bf16
    M, N, K = 4096 + 40, 2368, 264
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=85), rnd(N, K, dtype=torch.bfloat16, scale=0.1, seed=86)
    out = torch.zeros(M, N, device=DEV)
    assert kernels_bf16._tc_shape(M, N, out) == (256, 6, 2)
    assert kernels_bf16.linear_bf16(a, w, out, True)
    kernels_bf16.check_status()
    ref = a.double() @ w.double().T
    assert (out.double() - ref).abs().max().item() < 1e-5 * math.sqrt(K) * max(1.0, ref.abs().max().item())


def test_argmax_over_many_blocks():
    """Greedy over a large vocabulary (two-stage): ties across slices go to the lower id."""
    from gguf2bin_b200 import kernels
    R, V = 5, 151936
    logits = rnd(R, V, scale=2.0, seed=95)
    logits[1, 150000] = logits[1, 7] = 40.0
    logits[2, V - 1] = 41.0
    logits[3, 0] = 39.0
    ids = torch.empty(R, dtype=torch.int32, device=DEV)
    kernels.sample_rows(logits, 0.0, None, None, ids)
    assert ids.tolist() == [int(i) for i in logits.argmax(-1).tolist()][:1] + [7, V - 1, 0] + [int(logits[4].argmax())]
