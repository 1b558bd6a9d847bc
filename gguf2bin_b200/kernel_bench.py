"""Per-kernel micro-benchmarks at model geometry, in the manner of the reference's
tools/mmbench.c (which times its GEMV at the lm_head's size and prints GB/s): every hot
kernel alone, at the sizes of a decode step or of a prompt step, with its achieved
bandwidth or FLOP/s.

    python -m gguf2bin_b200.kernel_bench decode  [--batch 8] [--ctx 3072] [--only NAME] [--layers 28]
    python -m gguf2bin_b200.kernel_bench prefill [--tokens 2048] [--only NAME] [--layers 4]

Sizes default to Qwen3-0.6B (width 1024, 16/8 heads of 128, feed-forward 3072, vocabulary
151936); --hidden/--inter/--heads/--kv-heads/--vocab change them.  Decode kernels run
over `--layers` distinct weight sets, so weights stream from HBM as in a real step, and
are replayed from a CUDA graph; times are CUDA-event times per kernel launch.
`--only NAME --once` launches the named kernel a few times without graph or timing loop,
which is what a profiler capture wants.
"""
from __future__ import annotations

import argparse
import math
import sys
from types import SimpleNamespace

import torch

from . import kernels, kernels_bf16
from .engine.workspace import Workspace

DEV = "cuda:0"


def bf(*shape):
    return (torch.randn(*shape, device=DEV) * 0.02).to(torch.bfloat16)


class Bench:
    def __init__(self, a):
        self.a = a
        self.rows = []

    def want(self, name: str) -> bool:
        return self.a.only is None or self.a.only == name

    def run(self, name, fn, n_inner, nbytes=None, flops=None, graph=True):
        """Times `fn` (which launches the kernel n_inner times)."""
        if not self.want(name):
            return
        if self.a.once:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            print(f"{name}: launched 3 x {n_inner}")
            return
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        replay = fn
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            replay = g.replay
        replay()
        torch.cuda.synchronize()
        reps = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / reps / n_inner
        extra = ""
        if nbytes:
            extra += f"  {nbytes / us / 1e3:7.0f} GB/s"
        if flops:
            extra += f"  {flops / us / 1e6:7.0f} TFLOP/s"
        print(f"{name:28s} {us:9.2f} us{extra}")


def decode(a) -> None:
    B, L, H, I = a.batch, a.layers, a.hidden, a.inter
    nh, nkv, hd, V = a.heads, a.kv_heads, a.head_dim, a.vocab
    NQ, NK = nh * hd, nkv * hd
    b = Bench(a)
    x32 = torch.randn(B, H, device=DEV)
    nw = torch.ones(H, device=DEV)
    h, o, mid = bf(B, H), bf(B, NQ), bf(B, I)
    qkv = torch.empty(B, NQ + 2 * NK, dtype=torch.bfloat16, device=DEV)
    res = torch.zeros(B, H, device=DEV)
    hb = torch.empty(B, H, dtype=torch.bfloat16, device=DEV)
    b.run("rmsnorm", lambda: [kernels.rmsnorm(x32, nw, 1e-6, hb) for _ in range(L)], L)
    if b.want("qkv"):
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        b.run("qkv", lambda: [kernels_bf16.linear_bf16(h, w, qkv, False) for w in W], L, W[0].numel() * 2)
    if b.want("qkv_normed"):              # what a decode step of up to 16 rows runs: the norm inside the product
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        if kernels.normed_product(x32, 1e-6, W[0], qkv):
            b.run("qkv_normed", lambda: [kernels.normed_product(x32, 1e-6, w, qkv) for w in W], L, W[0].numel() * 2)
    if b.want("gate_up_normed"):
        W = [bf(2 * I, H) for _ in range(L)]
        if kernels.normed_product(x32, 1e-6, W[0], mid, 8):
            b.run("gate_up_normed", lambda: [kernels.normed_product(x32, 1e-6, w, mid, 8) for w in W], L,
                  W[0].numel() * 2)
    if b.want("o_proj"):
        W = [bf(H, NQ) for _ in range(L)]
        b.run("o_proj", lambda: [kernels_bf16.linear_bf16(o, w, res, True) for w in W], L, W[0].numel() * 2)
    if b.want("gate_up"):
        W = [bf(2 * I, H) for _ in range(L)]
        b.run("gate_up", lambda: [kernels_bf16.gate_up_bf16(h, w, mid, 8) for w in W], L, W[0].numel() * 2)
    if b.want("down"):
        W = [bf(H, I) for _ in range(L)]
        b.run("down", lambda: [kernels_bf16.linear_bf16(mid, w, res, True) for w in W], L, W[0].numel() * 2)
    if b.want("lm_head") or b.want("greedy") or b.want("temperature") or b.want("default_sampling"):
        from .cache import SEQ_STATE_WORDS
        Wh = bf(V, H)
        logits = torch.empty(B, V, device=DEV)
        ids = torch.empty(B, dtype=torch.int32, device=DEV)
        state = torch.zeros(B, SEQ_STATE_WORDS, dtype=torch.int32, device=DEV)
        slots = torch.arange(B, dtype=torch.int32, device=DEV)
        kernels.seed_slots(state, slots, slots.clone(), 1)
        b.run("lm_head", lambda: kernels_bf16.linear_bf16(h, Wh, logits, False), 1, Wh.numel() * 2)
        b.run("greedy", lambda: kernels.sample_rows(logits, 0.0, None, None, ids), 1, logits.numel() * 4)
        logits.copy_(torch.randn(B, V, device=DEV) * 2.5)
        b.run("temperature", lambda: kernels.sample_rows(logits, 0.7, state, slots, ids), 1, logits.numel() * 4)
        # temperature 0.7, top-k 40, top-p 0.9, repeat penalty 1.1 over the ids in the sequences' records
        b.run("default_sampling", lambda: kernels.sample_filtered(logits, 0.7, 40, 0.9, 1.1, None, None, state, slots,
                                                                  ids, append=True), 1, logits.numel() * 4)
    ps, ctx_len = 64, a.ctx
    pages_per = -(-(ctx_len + 1) // ps)
    if b.want("attn_decode") or b.want("qknorm_rope_cache"):
        caches = [torch.randn(B * pages_per, 2, nkv, ps, hd, device=DEV).to(torch.bfloat16) for _ in range(L)]
        table = torch.arange(B * pages_per, dtype=torch.int32, device=DEV).view(B, pages_per)
        ctx = SimpleNamespace(tok_pos=torch.full((B,), ctx_len, dtype=torch.int32, device=DEV),
                              tok_seq=torch.arange(B, dtype=torch.int32, device=DEV), page_table=table,
                              max_kv_len=pages_per * ps, workspace=Workspace(DEV), all_single=True)
        q = bf(B, NQ)
        out = torch.empty_like(q)
        b.run("attn_decode", lambda: [kernels_bf16.attn_decode(q, out, c, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd))
                                      for c in caches], L, B * (ctx_len + 1) * 2 * nkv * hd * 2)
        qw = torch.ones(hd, device=DEV)
        inv = torch.ones(hd // 2, device=DEV)
        rope = torch.empty(B, hd // 2, 2, device=DEV)
        kernels.rope_table(ctx.tok_pos, inv, rope)
        qkvb = bf(B, NQ + 2 * NK)
        b.run("qknorm_rope_cache", lambda: [kernels.qknorm_rope_cache(
            qkvb, nh, nkv, hd, qw, qw, 1e-6, rope, hd, ctx.tok_pos, ctx.tok_seq, table, c, ps, q) for c in caches], L)


def prefill(a) -> None:
    T, L, H, I = a.tokens, a.layers, a.hidden, a.inter
    nh, nkv, hd = a.heads, a.kv_heads, a.head_dim
    NQ, NK = nh * hd, nkv * hd
    b = Bench(a)
    x32 = torch.randn(T, H, device=DEV)
    nw = torch.ones(H, device=DEV)
    h, o, mid = bf(T, H), bf(T, NQ), bf(T, I)
    qkv = torch.empty(T, NQ + 2 * NK, dtype=torch.bfloat16, device=DEV)
    res = torch.zeros(T, H, device=DEV)
    hb = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    if b.want("qkv"):
        W = [bf(NQ + 2 * NK, H) for _ in range(L)]
        b.run("qkv", lambda: [kernels_bf16.linear_bf16(h, w, qkv, False) for w in W], L,
              flops=2 * T * (NQ + 2 * NK) * H)
    if b.want("o_proj"):
        W = [bf(H, NQ) for _ in range(L)]
        b.run("o_proj", lambda: [kernels_bf16.linear_bf16(o, w, res, True) for w in W], L,
              flops=2 * T * H * NQ)
    if b.want("gate_up"):
        W = [bf(2 * I, H) for _ in range(L)]
        b.run("gate_up", lambda: [kernels_bf16.gate_up_bf16(h, w, mid, 8) for w in W], L,
              flops=2 * T * 2 * I * H)
    if b.want("down"):
        W = [bf(H, I) for _ in range(L)]
        b.run("down", lambda: [kernels_bf16.linear_bf16(mid, w, res, True) for w in W], L,
              flops=2 * T * H * I)
    b.run("rmsnorm", lambda: [kernels.rmsnorm(x32, nw, 1e-6, hb) for _ in range(L)], L,
          nbytes=T * H * 6)
    ps = 64
    pages = -(-T // ps)
    if b.want("attn_prefill") or b.want("attn_prefill_tc") or b.want("qknorm_rope_cache"):
        caches = [torch.randn(pages, 2, nkv, ps, hd, device=DEV).to(torch.bfloat16) for _ in range(L)]
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
        tok_pos = torch.arange(T, dtype=torch.int32, device=DEV)
        tok_seq = torch.zeros(T, dtype=torch.int32, device=DEV)
        qw = torch.ones(hd, device=DEV)
        inv = (1e6 ** (-2 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
        q = bf(T, NQ)
        out = torch.empty_like(q)
        rope = torch.empty(T, hd // 2, 2, device=DEV)
        kernels.rope_table(tok_pos, inv, rope)
        b.run("qknorm_rope_cache", lambda: [kernels.qknorm_rope_cache(
            qkv, nh, nkv, hd, qw, qw, 1e-6, rope, hd, tok_pos, tok_seq, table, c, ps, q) for c in caches], L,
            nbytes=T * (NQ + 2 * NK) * 4)
        tiles = sorted([(0, r, min(64, T - r), r) for r in range(0, T, 64)], key=lambda t: -t[3])
        ctx = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles=len(tiles),
                              attn_tiles=torch.tensor(tiles, dtype=torch.int32, device=DEV))
        b.run("attn_prefill", lambda: [kernels_bf16.attn_prefill(q, out, c, ctx, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd))
                                       for c in caches], L, flops=4 * NQ * T * (T + 1) / 2)
        wide = sorted([(0, r, min(128, T - r), r) for r in range(0, T, 128)], key=lambda t: -t[3])
        ctx2 = SimpleNamespace(page_table=table, all_single=False, n_attn_tiles_wide=len(wide),
                               attn_tiles_wide=torch.tensor(wide, dtype=torch.int32, device=DEV))
        b.run("attn_prefill_tc", lambda: [kernels_bf16.attn_prefill_tc(
            q, out, c, ctx2, nh, nkv, hd, ps, 0, 1 / math.sqrt(hd)) for c in caches], L,
            flops=4 * NQ * T * (T + 1) / 2)
    kernels_bf16.check_status()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["decode", "prefill"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=3072)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--inter", type=int, default=3072)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--only", default=None, help="run one kernel by the name printed in the first column")
    ap.add_argument("--once", action="store_true", help="launch without graph or timing (for profilers)")
    a = ap.parse_args(argv)
    if a.layers is None:
        a.layers = 28 if a.mode == "decode" else 4
    (decode if a.mode == "decode" else prefill)(a)
    return 0


if __name__ == "__main__":
    sys.exit(main())
