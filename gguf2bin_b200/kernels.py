"""Python bindings of the CUDA kernels (ctypes over the C launchers of ``csrc/``).

Every function takes CUDA tensors, launches on the current torch stream and returns
nothing or its output tensor.  There is no CPU path: a tensor that is not on a CUDA
device raises ``KernelError``, and a missing or unbuildable extension raises
``KernelBuildError`` at the first call.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_ulonglong, c_void_p
from typing import Optional

import torch

from .csrc.build import KernelBuildError, KernelError, load_unit

__all__ = ["KernelError", "KernelBuildError", "embed_rows", "rmsnorm", "qknorm_rope_cache",
           "rope_table", "cache_write", "swiglu", "advance_positions", "gemm_simt", "linear", "attn_generic",
           "attention", "sample_rows", "sample_filtered", "recent_set", "seed_slots"]

F32, BF16 = 0, 1
EPI_STORE_F32, EPI_STORE_BF16, EPI_ACCUM_F32 = 0, 1, 2


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel called with a tensor that is not on a CUDA device "
                          "(there is no CPU path)")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """Handle of the current stream of the current device (the direct bindings when this
    torch has them: a launch costs microseconds on the host, and this is asked once per launch)."""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _need(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


_fn_cache: dict = {}
_bf16 = None              # the bfloat16 bindings (they import this module, so they are bound at first use)


def _bf16_mod():
    global _bf16
    if _bf16 is None:
        from . import kernels_bf16 as m
        _bf16 = m
    return _bf16


def _fn(unit: str, name: str, argtypes, defines=()):
    key = (unit, name, tuple(defines))
    f = _fn_cache.get(key)
    if f is None:
        lib = load_unit(unit, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        f._lib = lib
        _fn_cache[key] = f
    return f


_launches = 0
_scratch: dict = {}       # small persistent device buffers of the bindings, by (device, use)
_scratch_outgrown: list = []     # buffers that were replaced by larger ones: a captured graph may still use them


def _scratch_buffer(key, n: int, dtype) -> torch.Tensor:
    """The persistent buffer of that use with at least ``n`` elements.  A buffer that is
    outgrown is kept, not freed: launches captured in a CUDA graph go on writing to it."""
    buf = _scratch.get(key)
    if buf is None or buf.numel() < n or buf.dtype != dtype:
        if buf is not None:
            _scratch_outgrown.append(buf)
        buf = _scratch[key] = torch.empty(n, dtype=dtype, device=key[0])
    return buf


def launch_count() -> int:
    """How many kernels the launchers called so far in this process have launched."""
    return _launches


def count_launches(n: int) -> None:
    """A launcher that starts more than one kernel per call adds the others here."""
    global _launches
    _launches += n


def _call(f, *args) -> None:
    global _launches
    _launches += 1
    rc = f(*args)
    if rc != 0:
        raise KernelError(f._lib.g2b_last_error().decode("utf-8", "replace"))


# ---------------------------------------------------------------------------
# elementwise.cu
# ---------------------------------------------------------------------------
def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = table[ids[t]] widened to float32.  ids int32 [T], out float32 [T, H]."""
    _need(ids, torch.int32, "ids")
    _need(out, torch.float32, "out")
    V, H = table.shape
    f = _fn("elementwise.cu", "g2b_embed_rows",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _call(f, _ptr(table), _code(table.dtype), _ptr(ids), _ptr(out), out.shape[0], H, V, _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = (w * x[row_r]) / sqrt(mean(x[row_r]^2) + eps); x, w float32 (w None: all
    ones); statistics in float32.  ``rows`` (int32) gathers rows of x; out has one row per gathered row."""
    _need(x, torch.float32, "x")
    if w is not None:                      # None: no per-channel weight
        _need(w, torch.float32, "norm weight")
    if rows is not None:
        _need(rows, torch.int32, "rows")
    n_rows, H = out.shape
    f = _fn("elementwise.cu", "g2b_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p, c_int, c_void_p])
    _call(f, _ptr(x), _ptr(w), _ptr(rows), n_rows, H, eps, _ptr(out), _code(out.dtype), _stream())


def rope_table(tok_pos: torch.Tensor, inv_freq: torch.Tensor, table: torch.Tensor) -> None:
    """table[t, j] = (cos, sin)(tok_pos[t] * inv_freq[j]) in float32; table [T, half, 2]."""
    _need(tok_pos, torch.int32, "tok_pos")
    _need(inv_freq, torch.float32, "inv_freq")
    _need(table, torch.float32, "table")
    f = _fn("elementwise.cu", "g2b_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _call(f, _ptr(tok_pos), _ptr(inv_freq), _ptr(table), table.shape[0], inv_freq.shape[0], _stream())


def qknorm_rope_cache(qkv, n_heads, n_kv_heads, head_dim, q_w, k_w, eps, rope, rotary_dim,
                      tok_pos, tok_seq, page_table, cache_pages, page_size, q_out,
                      k_out=None, v_out=None) -> None:
    """Per-head RMSNorm of the q and k heads (when q_w / k_w are given), half-split
    rotation by the angles of ``rope`` (a table from ``rope_table`` for this step's
    tokens; None: no rotation), q to ``q_out``; k and v to the layer's cache pages, or to
    ``k_out`` / ``v_out`` when those are given."""
    T = qkv.shape[0]
    f = _fn("elementwise.cu", "g2b_qknorm_rope_cache",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
             c_void_p, c_void_p])
    P = page_table.shape[1] if page_table is not None else 0
    for t in (q_out, k_out, v_out, cache_pages):
        if t is not None and t.dtype != qkv.dtype:
            raise KernelError("qknorm_rope_cache: outputs and cache must have the input's dtype")
    _call(f, _ptr(qkv), _code(qkv.dtype), T, n_heads, n_kv_heads, head_dim, _ptr(q_w), _ptr(k_w),
          eps, _ptr(rope), rotary_dim, _ptr(tok_pos), _ptr(tok_seq), _ptr(page_table), P,
          _ptr(cache_pages), page_size, _ptr(q_out), _ptr(k_out), _ptr(v_out), _stream())


def cache_write(k, v, n_kv_heads, head_dim, tok_pos, tok_seq, page_table, cache_pages,
                page_size) -> None:
    """k, v [T, n_kv_heads*head_dim] into the layer's cache pages at each token's position."""
    f = _fn("elementwise.cu", "g2b_cache_write",
            [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
             c_void_p, c_int, c_void_p])
    if k.dtype != cache_pages.dtype or v.dtype != cache_pages.dtype:
        raise KernelError("cache_write: k, v and the cache must have one dtype")
    _call(f, _ptr(k.contiguous()), _ptr(v.contiguous()), _code(k.dtype), k.shape[0], n_kv_heads,
          head_dim, _ptr(tok_pos), _ptr(tok_seq), _ptr(page_table), page_table.shape[1],
          _ptr(cache_pages), page_size, _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int) -> None:
    """out[t, i] = silu(g_i) * u_i from a fused projection whose columns alternate
    ``block`` gates and ``block`` ups."""
    T, I = out.shape
    f = _fn("elementwise.cu", "g2b_swiglu",
            [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
    _call(f, _ptr(gate_up), _code(gate_up.dtype), T, I, block, _ptr(out), _stream())


def advance_positions(tok_pos: torch.Tensor, n: int) -> None:
    f = _fn("elementwise.cu", "g2b_advance_positions", [c_void_p, c_int, c_void_p])
    _call(f, _ptr(tok_pos), n, _stream())


def rewind_step(tok_pos: torch.Tensor, n: int, seq_state: Optional[torch.Tensor], slots: Optional[torch.Tensor],
                undo_draw: bool, undo_recent: bool = False) -> None:
    """Takes back the device-side bookkeeping of one decode step (positions; the draw
    counters of the sampling records when that step sampled with a random number; the count
    of recent ids when it added one to the sequences' rings)."""
    f = _fn("elementwise.cu", "g2b_rewind_step",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    words = seq_state.shape[1] if seq_state is not None else 0
    _call(f, _ptr(tok_pos), n, _ptr(seq_state), words, _ptr(slots), 1 if undo_draw else 0,
          1 if undo_recent else 0, _stream())


# ---------------------------------------------------------------------------
# random_init.cu
# ---------------------------------------------------------------------------
def philox_normal(out: torch.Tensor, seed: int, tensor_index: int, scale_vector: bool, std: float) -> None:
    """Fills ``out`` (float32 or bfloat16, contiguous) in place with N(0, std), or with
    1 + N(0, std) for a scale vector; element i gets the value of (seed, tensor_index, i)."""
    if not out.is_contiguous():
        raise KernelError("philox_normal: the tensor must be contiguous")
    from ctypes import c_longlong, c_uint
    f = _fn("random_init.cu", "g2b_philox_normal",
            [c_void_p, c_int, c_longlong, c_ulonglong, c_uint, c_int, c_float, c_void_p])
    _call(f, _ptr(out), _code(out.dtype), out.numel(), int(seed) & 0xFFFFFFFFFFFFFFFF,
          int(tensor_index) & 0xFFFFFFFF, 1 if scale_vector else 0, float(std), _stream())


# ---------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (=|+=) a @ w.T in true float32 arithmetic.  a [M,K], w [N,K], out [M,N];
    accumulate needs a float32 out."""
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: shapes a{list(a.shape)} w{list(w.shape)} out{list(out.shape)}")
    if accumulate:
        _need(out, torch.float32, "accumulated output")
        epi = EPI_ACCUM_F32
    else:
        epi = EPI_STORE_F32 if out.dtype == torch.float32 else EPI_STORE_BF16
        _code(out.dtype)
    f = _fn("gemm_simt.cu", "g2b_gemm_simt",
            [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
             c_int, c_void_p])
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm: innermost strides must be 1")
    _call(f, _ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), _ptr(out), M, N, K, a.stride(0),
          w.stride(0), out.stride(0), epi, _stream())


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """The product a layer asks for; picks the kernel from the dtypes and sizes.  Anything
    that is not all-bfloat16 runs on the float32 kernel (true 32-bit arithmetic)."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        if (_bf16 or _bf16_mod()).linear_bf16(a, w, out, accumulate):
            return
    gemm_simt(a, w, out, accumulate)


def product_notices(what: str, w: Optional[torch.Tensor], compute_dtype: torch.dtype) -> list:
    """Why products with the matrix ``w`` will run on the 32-bit FFMA kernel although the
    model computes in bfloat16: one line per reason, for the notice printed when a model is
    built (the result is right either way; the speed is not the same)."""
    if w is None or compute_dtype != torch.bfloat16:
        return []
    if w.dtype != torch.bfloat16:
        return [f"{what}: the matrix is kept in {str(w.dtype).replace('torch.', '')} as stored, so its "
                "products run on the 32-bit FFMA kernel, not on the tensor cores"]
    if w.shape[1] % 8 or w.stride(0) % 8 or w.data_ptr() % 16:
        return [f"{what}: K = {w.shape[1]} is no multiple of 8, so its products run on the 32-bit "
                "FFMA kernel, not on the tensor cores"]
    return []


def attention_notices(what: str, head_dim: int, page_size: int, compute_dtype: torch.dtype) -> list:
    if compute_dtype != torch.bfloat16:
        return []
    from . import kernels_bf16
    if head_dim not in kernels_bf16.FAST_HEAD_SIZES or page_size != 64:
        sizes = " and ".join(str(h) for h in kernels_bf16.FAST_HEAD_SIZES)
        return [f"{what}: head size {head_dim} runs on the 32-bit attention kernel (the tensor-core "
                f"kernels take head sizes {sizes})"]
    return []


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def attn_generic(q, out, cache_pages, tok_pos, tok_seq, page_table, n_heads, n_kv_heads,
                 head_dim, page_size, window, scale) -> None:
    """Causal attention of every token of the step over its sequence's cache pages,
    32-bit arithmetic; q, out [T, n_heads*head_dim]."""
    f = _fn("attn_generic.cu", "g2b_attn_generic",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
             c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    if q.dtype != cache_pages.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, out and the cache must have one dtype")
    _call(f, _ptr(q), _ptr(out), _code(q.dtype), _ptr(cache_pages), _ptr(tok_pos), _ptr(tok_seq),
          _ptr(page_table), page_table.shape[1], q.shape[0], n_heads, n_kv_heads, head_dim,
          page_size, window, scale, _stream())


def attention(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim, page_size, window,
              scale) -> None:
    """Attention of a step: the tensor-core kernels when they take the case, else the
    32-bit kernel."""
    if q.dtype == torch.bfloat16:
        if (_bf16 or _bf16_mod()).attention_bf16(q, out, cache_pages, ctx, n_heads, n_kv_heads, head_dim,
                                       page_size, window, scale):
            return
    attn_generic(q, out, cache_pages, ctx.tok_pos, ctx.tok_seq, ctx.page_table, n_heads,
                 n_kv_heads, head_dim, page_size, window, scale)


def normed_product(x32, eps, w, out, gate_block=None) -> bool:
    """out = rmsnorm_without_weight(x32) @ w.T (or its SiLU gate) in one kernel; False when no
    kernel takes the case (the caller then runs the norm and the product one after the other)."""
    if w.dtype == torch.bfloat16 and (gate_block is None or gate_block == 8):
        return (_bf16 or _bf16_mod()).normed_product(x32, eps, w, out, gate_block is not None)
    return False


def gate_up_fused(h, w_gate_up, mid, block) -> bool:
    """silu(gate) * up computed inside the product's epilogue; False when no kernel takes
    the case (the caller then runs the product and ``swiglu`` separately)."""
    if h.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16:
        return (_bf16 or _bf16_mod()).gate_up_bf16(h, w_gate_up, mid, block)
    return False


# ---------------------------------------------------------------------------
# sampling.cu
# ---------------------------------------------------------------------------
def sample_rows(logits, temperature, seq_state, slots, out_ids) -> None:
    """Greedy (temperature <= 0) or temperature sampling of one id per row of float32
    logits; random numbers come from the per-slot records."""
    _need(logits, torch.float32, "logits")
    _need(out_ids, torch.int32, "out_ids")
    R, V = logits.shape
    if temperature <= 0.0 and V >= 4096:
        # greedy over a large vocabulary: many blocks per row, then one
        n = max(R, 64) * 64
        scratch = (_scratch_buffer((logits.device, "argmax values"), n, torch.float32),
                   _scratch_buffer((logits.device, "argmax indices"), n, torch.int32))
        f = _fn("sampling.cu", "g2b_argmax_rows",
                [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
        _call(f, _ptr(logits), R, V, logits.stride(0), _ptr(scratch[0]), _ptr(scratch[1]),
              _ptr(out_ids), _stream())
        count_launches(1)                          # the slices, then the winner among them
        return
    f = _fn("sampling.cu", "g2b_sample_rows",
            [c_void_p, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p])
    pieces = None
    if temperature > 0.0 and V >= 8192:
        # a large vocabulary: many blocks per row sum its pieces first
        pieces = _scratch_buffer((logits.device, "pieces"), max(R, 64) * 2048 * 2, torch.float32)
        count_launches(1)
    _call(f, _ptr(logits), R, V, logits.stride(0), temperature, _ptr(seq_state),
          seq_state.shape[1] if seq_state is not None else 0, _ptr(slots), _ptr(out_ids), _ptr(pieces),
          _stream())


def sample_filtered(logits, temperature, top_k, top_p, penalty, recent, recent_n, seq_state, slots,
                    out_ids, append: bool = False) -> None:
    """Repeat penalty, top-k, top-p, then temperature sampling; logits are changed in
    place by the penalty.  recent int32 [R, n], recent_n int32 [R]; or ``recent=None``: every
    row's recent ids are those in its sequence's record (``seq_state[slots[row]]``), to which
    the chosen id is added when ``append`` is set."""
    _need(logits, torch.float32, "logits")
    _need(out_ids, torch.int32, "out_ids")
    R, V = logits.shape
    if recent is not None:
        _need(recent, torch.int32, "recent")
        _need(recent_n, torch.int32, "recent_n")
        if recent.shape[0] < R or recent_n.shape[0] < R:
            raise KernelError("sample_filtered: recent and recent_n need a row per row of logits")
    f = _fn("sampling.cu", "g2b_sample_filtered",
            [c_void_p, c_int, c_int, c_int, c_float, c_int, c_float, c_float, c_void_p, c_int,
             c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p])
    cand = None
    if temperature > 0.0 and 0 < top_k <= 256 and V >= 8192:
        # a small top_k over a large vocabulary: many blocks per row list the candidates first
        words = _fn("sampling.cu", "g2b_sample_filtered_scratch_words", [c_int])
        cand = _scratch_buffer((logits.device, "filter"), int(words(max(R, 64))), torch.int32)
        count_launches(1)
    _call(f, _ptr(logits), R, V, logits.stride(0), temperature, top_k, top_p, penalty,
          _ptr(recent), recent.shape[1] if recent is not None else 0, _ptr(recent_n),
          _ptr(seq_state), seq_state.shape[1] if seq_state is not None else 0, _ptr(slots),
          _ptr(out_ids), 1 if append else 0, _ptr(cand), _stream())


def recent_set(seq_state, slots, rows) -> None:
    """Starts the recent-id rings of the given slots: rows int32 [n, 65] = count, ids (oldest
    first); the repeat penalty of later ``sample_filtered`` calls without ``recent`` reads them."""
    _need(slots, torch.int32, "slots")
    _need(rows, torch.int32, "rows")
    if rows.dim() != 2 or rows.shape[1] != 65 or rows.shape[0] < slots.shape[0]:
        raise KernelError("recent_set: rows must be [n, 65]")
    f = _fn("sampling.cu", "g2b_recent_set", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _call(f, _ptr(seq_state), seq_state.shape[1], _ptr(slots), _ptr(rows), slots.shape[0], _stream())


def seed_slots(seq_state, slots, streams, seed: int) -> None:
    """Starts the random stream of each given slot: key = seed, stream id, zero draws."""
    f = _fn("sampling.cu", "g2b_seed_slots",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_ulonglong, c_void_p])
    _call(f, _ptr(seq_state), seq_state.shape[1], _ptr(slots), _ptr(streams), slots.shape[0],
          seed & 0xFFFFFFFFFFFFFFFF, _stream())
