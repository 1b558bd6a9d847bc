"""Bindings of the bfloat16 tensor-core kernels.  Each function returns True when it ran,
False when it does not take the case (the caller then uses the 32-bit kernel)."""
from __future__ import annotations

from ctypes import c_longlong, c_float, c_int, c_void_p

import torch

from .csrc import units
from . import kernels
from .kernels import KernelError, _call, _fn, _ptr, _stream

FAST_HEAD_SIZES = (64, 128)          # head sizes the tensor-core attention kernels are written for
DECODE_CHUNK_KEYS = 256              # keys per CTA of the decode kernel (attn_decode.cu)

units.SPECIALISED_SOURCES[:] = [("attn_decode.cu", ()), ("attn_decode.cu", ("ATTN_DECODE_PAGES=2",)),
                                ("attn_decode.cu", ("ATTN_DECODE_PAGES=6",)), ("attn_decode.cu", ("ATTN_DECODE_PAGES=8",)),
                                ("attn_decode_noalloc.cu", ()),
                                ("attn_prefill.cu", ()), ("attn_prefill_tc.cu", ()),
                                ("attn_prefill_tc_split.cu", ())]
units.BF16_UNITS[:] = [("gemm_small.cu", ()), ("gemm_tc.cu", ())]


SMALL_M = 64                         # rows the weight-streaming product takes
EPI_STORE_BF16, EPI_STORE_F32, EPI_ACCUM_F32, EPI_SWIGLU_BF16 = 0, 1, 2, 3


def _small_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    K = a.shape[1]
    return (a.shape[0] <= SMALL_M and K % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _gemm_small(a, w, out, epi) -> None:
    f = _fn("gemm_small.cu", "g2b_gemm_small",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _call(f, _ptr(a), _ptr(w), _ptr(out), a.shape[0], w.shape[0], a.shape[1], a.stride(0),
          w.stride(0), out.stride(0), epi, _stream())


def normed_product(x32: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor, gated: bool) -> bool:
    """out = rmsnorm(x32) @ w.T for the float stream x32 [M, K] with a weightless RMS norm
    (x / sqrt(mean(x^2) + eps)) computed inside the few-row product: the row's factor scales
    the accumulators.  ``gated``: w is a fused gate/up matrix (rows alternating 8 / 8) and out
    gets silu(gate) * up.  False when the case is not taken (more than 16 rows, a K that is
    split over a cluster or streamed in chunks, or a case that a norm kernel and the tcgen05 product do
    faster: ``_normed_loses``)."""
    M, K = x32.shape
    N = w.shape[0]
    if (x32.dtype != torch.float32 or w.dtype != torch.bfloat16 or x32.stride(1) != 1 or w.stride(1) != 1
            or out.stride(1) != 1 or x32.stride(0) % 4 or w.stride(0) % 8
            or x32.data_ptr() % 16 or w.data_ptr() % 16):
        return False
    if gated:
        if out.dtype != torch.bfloat16 or N % 16:
            return False
        epi = EPI_SWIGLU_BF16
    elif out.dtype == torch.bfloat16:
        epi = EPI_STORE_BF16
    elif out.dtype == torch.float32:
        epi = EPI_STORE_F32
    else:
        return False
    if _normed_loses(M, N, K):
        return False
    takes = _fn("gemm_small.cu", "g2b_gemm_small_normed_takes", [c_int, c_int, c_int])
    if not takes(M, N, K):
        return False
    f = _fn("gemm_small.cu", "g2b_gemm_small_normed",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _call(f, _ptr(x32), _ptr(w), _ptr(out), M, N, K, x32.stride(0), w.stride(0), out.stride(0), epi,
          float(eps), _stream())
    return True


_status: dict = {}


def _status_word(device) -> torch.Tensor:
    """The device word in which the tcgen05 kernels report a wait that gave up."""
    word = _status.get(device)
    if word is None:
        key = torch.device(device)
        if key not in _status:
            _status[key] = torch.zeros(1, dtype=torch.int32, device=key)
        word = _status[key]
    return word


def check_status() -> None:
    """Raises if a kernel's bounded wait gave up since the last check (reads the device
    word, so it synchronises)."""
    for dev, word in _status.items():
        code = int(word.item())
        if code:
            word.zero_()
            if code == 14:
                raise KernelError(f"attn_prefill_tc on {dev}: dynamic shared memory does not start on a "
                                  "1024-byte boundary; nothing was computed")
            kernel = "attn_prefill_tc" if code > 10 else "gemm_tc"
            what = {1: "the TMA producer", 2: "the MMA issuer", 3: "the epilogue",
                    4: "a CTA of a pair, for its peer at the end of the kernel,",
                    11: "the TMA producer", 12: "the MMA issuer", 13: "a softmax warp"}.get(code, "a role")
            raise KernelError(f"{kernel} on {dev}: {what} gave up waiting on a barrier (code {code}); "
                              "the result of that launch is invalid")


def _tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    K = a.shape[1]
    return (K % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1 and a.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def _gemm_tc(a, w, out, epi, bn: int = 0, stages: int = 0, persistent=False, defines=()) -> None:
    """bn = 0 lets the launcher pick the tile shape from the sizes.  persistent: one CTA per SM
    walks over the tiles with two accumulators (shapes (128, 6) and (256, 4)); persistent = 2:
    pairs of CTAs on 256 x 256 tiles (shapes (256, 6) and (256, 4)); persistent = 3: at most 128
    rows, 128 rows of W per CTA and K split over a cluster (bn and stages are not used).
    ``defines``: another build of the source (the tests' build whose waits run out)."""
    f = _fn("gemm_tc.cu", "g2b_gemm_tc",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_int, c_void_p, c_void_p], defines=tuple(defines))
    _call(f, _ptr(a), _ptr(w), _ptr(out), a.shape[0], w.shape[0], a.shape[1], a.stride(0),
          w.stride(0), out.stride(0), epi, bn, stages, int(persistent),
          _ptr(_status_word(a.device)), _stream())


_routes: dict = {}        # (sizes, strides, alignment, output) -> (kernel, tile width, stages, persistent)


def _route(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor):
    """Which kernel multiplies a by w.T into out, and with which tile shape: decided once per
    combination of sizes, strides and alignments (a step asks the same few questions a hundred
    times, and on a prompt's first run the host is what the GPU waits for)."""
    key = (a.shape, w.shape, a.stride(), w.stride(), out.stride(), out.dtype,
           (a.data_ptr() | w.data_ptr()) & 15, out.data_ptr() & 15, out.device.index)
    r = _routes.get(key)
    if r is None:
        choice = _pick_product(a, w)
        shape = _tc_shape(a.shape[0], w.shape[0], out, a.shape[1]) if choice == "tc" else (0, 0, False)
        if len(_routes) > 4096:
            _routes.clear()
        r = _routes[key] = (choice,) + tuple(shape)
    return r


def linear_bf16(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool) -> bool:
    """out (=|+=) a @ w.T for bfloat16 a and w on the tensor cores."""
    choice, bn, stages, persistent = _route(a, w, out)
    if out.stride(1) != 1:
        return False
    if accumulate:
        if out.dtype != torch.float32:
            return False
        epi = EPI_ACCUM_F32
    else:
        epi = EPI_STORE_BF16 if out.dtype == torch.bfloat16 else EPI_STORE_F32
    if choice == "small":
        _gemm_small(a, w, out, epi)
        return True
    if choice == "tc":
        _gemm_tc(a, w, out, epi, bn, stages, persistent)
        return True
    return False


def _pick_product(a: torch.Tensor, w: torch.Tensor):
    """Which kernel multiplies: the weight-streaming mma.sync one up to 16 rows, and up to 64
    for narrow outputs, wherever the tcgen05 kernel with K split over a cluster was not measured
    faster (``_wstream_case``); the tcgen05 ones otherwise."""
    M, N, K = a.shape[0], w.shape[0], a.shape[1]
    small, tc_ = _small_ok(a, w), _tc_ok(a, w)
    if small and (not tc_ or (not _wstream_case(M, N, K) and (M <= 16 or (M <= SMALL_M and N <= 2048)))):
        return "small"
    if tc_:
        return "tc"
    return None


def _wstream_case(M: int, N: int, K: int) -> bool:
    """Few rows whose product goes to the kernel with 128 rows of W per CTA and K split over a
    cluster.  Against big weights (N and K of 2,048 and more), measured at the layer sizes of
    Qwen3-1.7B to 14B: from 9 to 64 rows (10.7 against 13.4 us by the mma.sync kernel for
    4096 x 4096 at 16 rows) unless the matrix is small (4096 x 2048 at 16 rows: 7.2 against 5.5 us;
    2048 x 2048 at 32 rows: 6.0 against 5.3); up to 8 rows only against the largest matrices or a
    very long K (5120 x 17408: 31.6 against 43.8 us; 2048 x 6144: 10.7 against 17.0; but
    6144 x 4096: 13.4 against 12.3, and the mma.sync kernel can take the norm in front along);
    from 65 rows only narrow outputs up to 96 rows (24576 x 4096 at 65 rows: 54.0 against 39.0 us
    by the persistent kernel; 4096 x 12288: 22.8 against 24.7).
    A vocabulary (151,936 rows) at every number of rows up to 64: at K = 2,048 to 5,120 it reads
    W at 6.2-6.4 TB/s with 1 to 8 rows where the mma.sync kernel reaches 5.5-6.3 (K = 2,048, one row:
    97.8 against 108.5 us), and at 16 rows and more the other kernels are far behind (K = 4,096,
    16 rows: 200 against 584 us).  At K = 1,024 from 9 rows (16 rows: 56.2 against 81.8 us; 64 rows:
    64.4 against 81.2 by 128 x 128 tiles, one per CTA); up to 8 rows the two are within 4 us and the
    mma.sync kernel takes the final norm along.
    Against the weights of a small model's layers from 17 rows where it was measured faster
    (at 64 rows, 1024 x 3072: 8.5 us against 17.8 by the mma.sync kernel and 18.4 by one
    128 x 64 tile per CTA); wide outputs with K = 1024 up to 48 rows, or 64 with 4,096 outputs
    (6144 x 1024 at 48 rows: 7.8 against 9.0 us by 128 x 64 tiles, at 64 rows 8.4 against 8.0; at
    128 rows: 11.7 us against 8.4)."""
    if M > 128:
        return False
    if N >= 2048 and K >= 2048:
        if M <= 8:
            return N * K > (24 << 20) or K >= 6144
        if M <= 16:
            return N * K > (8 << 20)
        if M <= 32:
            return N * K > (4 << 20)
        if M <= 64:
            return True
        return N < 8192 and M <= 96
    if N > 65536:                      # a vocabulary with a short K
        return 8 < M <= 64 and K >= 1024
    if M <= 16 or N < 1024 or K < 1024 or N > 16384:
        return False
    if N < 2048:                       # narrow outputs: 1024 x 2048 at 32 rows is 4.9 us by the mma.sync kernel, 6.6 here
        return not (M <= 32 and K <= 2048)
    return M <= 48 or (M <= 64 and N <= 4096)      # wide outputs with a short K


def _normed_loses(M: int, N: int, K: int) -> bool:
    """Whether the few-row product that takes the norm along is the slower way: 9 to 16 rows
    against big weights (a decode step of 16 sequences at Qwen3-8B sizes: 270 us a layer with it,
    160 with a norm kernel and the tcgen05 product), and up to 8 rows against the largest
    matrices, a vocabulary among them (34816 x 5120: 62.4 us against 54.6 + 2.1)."""
    if N < 2048 or K < 2048:
        return False
    if M > 8:
        return True
    return N * K >= (48 << 20)


def _tc_shape(M: int, N: int, out: torch.Tensor = None, K: int = 0):
    """(tile width, stages, persistent) of the tcgen05 product; (0, 0, False) lets the launcher
    choose.  Prompts (more than one row of tiles) take the persistent kernel when C can be
    written as tiles (the launcher picks the tile width, and with few tiles K in parts); long prompts
    take pairs of CTAs (persistent = 2; measured 4-9 % faster from 4,096 rows on, the same or
    slower at 2,048 with the short K of a small model; with a K of 4,096 and more from 1,024 rows on)."""
    if M <= 128:                       # one row of tiles: the weights stream, as in decode
        if _wstream_case(M, N, K):
            return (0, 0, 3)           # 128 rows of W per CTA, K split over a cluster
        if not (M > 64 and N >= 2048 and K >= 2048 and N <= 65536):      # (else the persistent kernel, below)
            return (128, 3, False) if N >= 32768 else (64, 8, False)
    if out is not None and out.data_ptr() % 16 == 0 and (out.stride(0) * out.element_size()) % 16 == 0:
        tiles = -(-M // 256) * -(-N // 256)
        if M >= 4096 and tiles >= _sm_count(out.device) // 2:
            return (256, 6, 2)               # long prompts: pairs of CTAs on 256 x 256 tiles
        if M >= 1024 and K >= 4096 and tiles >= 48:
            # A long K (the layer sizes of Qwen3-8B and 14B) from 1,024 rows on: 3 to 9 % faster than the
            # persistent kernel at 1,024 to 3,072 rows (6144 x 4096 at 2,048 rows: 70.4 against 74.9 us;
            # 4096 x 12288: 143.9 against 154.3), 5120 x 17408 at 2,048 rows 279 against 392 us; only
            # 24576 x 4096 at 3,072 rows lost 2 %.  With K up to 3,072 (a small model) it was the same or slower.
            return (256, 6, 2)
        return (0, 0, True)                  # the launcher picks the width and, with few tiles, parts of K
    return (0, 0, False)


_sm_counts: dict = {}


def _sm_count(device) -> int:
    key = torch.device(device)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


def gate_up_bf16(h: torch.Tensor, w_gate_up: torch.Tensor, mid: torch.Tensor, block: int) -> bool:
    """mid = silu(gate) * up with the gate computed in the product's epilogue; takes fused
    matrices whose rows alternate 8 gates / 8 ups."""
    if block != 8 or mid.dtype != torch.bfloat16 or mid.stride(1) != 1 or w_gate_up.shape[0] % 16:
        return False
    choice, bn, stages, persistent = _route(h, w_gate_up, mid)
    if choice == "small":
        _gemm_small(h, w_gate_up, mid, EPI_SWIGLU_BF16)
        return True
    if choice == "tc":
        _gemm_tc(h, w_gate_up, mid, EPI_SWIGLU_BF16, bn, stages, persistent)
        return True
    return False


def attention_bf16(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
                   scale) -> bool:
    if head_dim not in FAST_HEAD_SIZES or page_size != 64 or cache_pages.dtype != torch.bfloat16:
        return False
    if ctx.all_single:
        attn_decode(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window, scale)
        return True
    if USE_TC_ATTENTION and getattr(ctx, "attn_tiles_wide", None) is not None and ctx.n_attn_tiles_wide > 0:
        attn_prefill_tc(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window, scale)
        return True
    if getattr(ctx, "attn_tiles", None) is not None and ctx.n_attn_tiles > 0:
        attn_prefill(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window, scale)
        return True
    return False


USE_TC_ATTENTION = True      # prompt attention on tcgen05 (else the mma.sync kernel)


def attn_prefill_tc(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
                    scale, defines=(), split=None) -> None:
    """Prompt attention on the tcgen05 tensor cores over the step's 128-row query tiles.  Two
    kernels with the same interface: two CTAs per SM, a tile each (``attn_prefill_tc.cu``), and
    one CTA per SM whose two softmax groups share a tile's pages (``attn_prefill_tc_split.cu``;
    ``split``).  The second by default when the work list is at most one item (tile x head) per SM,
    or at most two per SM with tiles of a thousand keys and more: 16 heads at 2,048 tokens 26.8
    against 32.6 us, 1,536 tokens 18.6 against 24.2, 32 heads at 512 tokens 10.0 against 11.5; but
    eight prompts of 256 tokens (256 items of two and four pages) 14.0 against 10.5 by two CTAs per
    SM, and 160 items of up to eight pages 14.1 against 12.5.
    ``defines``: another build of the source (the tests' build whose waits run out)."""
    if split is None:
        items, sms = ctx.n_attn_tiles_wide * n_heads, _sm_count(q.device)
        split = items <= sms or (items <= 2 * sms and getattr(ctx, "max_kv_len", 0) >= 1024)
    f = _fn("attn_prefill_tc_split.cu" if split else "attn_prefill_tc.cu", "g2b_attn_prefill_tc",
            [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
            defines=(f"HD={head_dim}",) + tuple(defines))
    _call(f, _ptr(q), _ptr(out), _ptr(cache_pages), cache_pages.shape[0], _ptr(ctx.attn_tiles_wide),
          ctx.n_attn_tiles_wide, _ptr(ctx.page_table), ctx.page_table.shape[1], q.shape[0], n_heads,
          n_kv_heads, head_dim, page_size, window, scale, _ptr(_status_word(q.device)), _stream())


def attn_prefill(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
                 scale) -> None:
    """Prompt attention over the step's work list of 64-row query tiles."""
    f = _fn("attn_prefill.cu", "g2b_attn_prefill",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
             c_int, c_int, c_float, c_void_p], defines=(f"HD={head_dim}",))
    _call(f, _ptr(q), _ptr(out), _ptr(cache_pages), _ptr(ctx.attn_tiles), ctx.n_attn_tiles,
          _ptr(ctx.page_table), ctx.page_table.shape[1], n_heads, n_kv_heads, head_dim, page_size,
          window, scale, _stream())


DECODE_FINE_BELOW = 200       # CTAs of 256-key chunks below which the chunks are halved (measured: two sequences)
DECODE_CTAS_PER_SM = 3        # CTAs of the decode kernel that an SM holds at head size 128 (64 KB of panels each)


def decode_chunk_pages(units: int, pages: int, head_dim: int, slots: int) -> int:
    """Pages of 64 keys per CTA of the decode attention: 4 (chunks of 256 keys) as a rule; 2
    when that gives fewer CTAs than the GPU holds at once (one or two sequences); 6 or 8 when
    the CTAs of 4 pages come in one round and a bit (8 sequences at 2,048 to 2,300 keys: 512 to
    576 CTAs for 444 places took 16.5 to 17.2 us, 384 CTAs at 1,536 keys 11.8) and longer chunks
    make it fewer rounds' worth of pages.  ``units``: tokens x kv heads x head tiles;
    ``slots``: CTAs the GPU holds at once."""
    ctas4 = units * -(-pages // 4)
    if ctas4 < DECODE_FINE_BELOW:
        return 2
    best, cost = 4, -(-ctas4 // slots) * 4
    if head_dim == 128:
        for ppc in (6, 8):
            c = -(-(units * -(-pages // ppc)) // slots) * ppc
            if c < cost:
                best, cost = ppc, c
    return best


def attn_decode(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
                scale, fine=None, pages=None) -> None:
    """One token per sequence: split-key attention with partial results in scratch memory
    and a combine pass.  A CTA takes a chunk of keys of one kv head: 256 as a rule, 128, 384 or
    512 where ``decode_chunk_pages`` says so (``fine`` = 128; ``pages`` = pages of 64 keys per
    CTA, 2 to 8; default by that rule)."""
    T = q.shape[0]
    defines = (f"HD={head_dim}",)
    if pages is None:
        if fine is None:
            tiles = n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
            keys = getattr(ctx, "kv_len_hint", 0) or ctx.max_kv_len       # max_kv_len may be the reserved length
            pages = decode_chunk_pages(T * tiles, -(-max(int(keys), 1) // 64), head_dim,
                                       DECODE_CTAS_PER_SM * _sm_count(q.device))
        else:
            pages = 2 if fine else 4
    if pages != 4:
        defines = defines + (f"ATTN_DECODE_PAGES={pages}",)
    chunk_keys = 64 * pages
    n_chunks = -(-max(int(ctx.max_kv_len), 1) // chunk_keys)
    ws = ctx.workspace
    part_o = ws.buffer("attn.part_o", (T * n_heads * n_chunks * head_dim,), torch.float32)
    part_ml = ws.buffer("attn.part_ml", (T * n_heads * n_chunks * 2,), torch.float32)
    f = _fn("attn_decode.cu", "g2b_attn_decode",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p],
            defines=defines)
    _call(f, _ptr(q), _ptr(out), _ptr(cache_pages), _ptr(ctx.tok_pos), _ptr(ctx.tok_seq),
          _ptr(ctx.page_table), ctx.page_table.shape[1], T, n_heads, n_kv_heads, head_dim,
          page_size, window, scale, int(ctx.max_kv_len), _ptr(part_o), _ptr(part_ml), _stream())
    kernels.count_launches(1)                      # the attention and the merge of its chunks
