"""Plain, slow restatement of the Qwen3 dense forward pass, for tests only.

Written from the formulas of AnonymoDGH/gguf2bin (file:line cited on every
function; paths are relative to that project).  Whole sequences, no cache, one
function per part, numpy only.  It shares no code with ``gguf2bin_b200``: it has
its own safetensors reader, its own configuration reading and its own sampler.

The arithmetic dtype is a parameter (float32 as the reference computes, or
float64 for a rounding-free truth).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np


# ----------------------------------------------------------------------------
# model folder reading (own code; the product's loader is not used)
# ----------------------------------------------------------------------------
_ST_DTYPES = {"F32": np.float32, "F16": np.float16, "F64": np.float64,
              "I32": np.int32, "I64": np.int64}


def _bf16_to_f32(raw: bytes) -> np.ndarray:
    u16 = np.frombuffer(raw, dtype="<u2").astype(np.uint32)
    return (u16 << 16).view(np.float32)


def read_safetensors(path) -> dict:
    """name -> float32/int ndarray.  Format: 8-byte LE header length, JSON header
    (name -> dtype, shape, data_offsets), raw little-endian data."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        raw = blob[base + a: base + b]
        if info["dtype"] == "BF16":
            arr = _bf16_to_f32(raw)
        else:
            arr = np.frombuffer(raw, dtype=np.dtype(_ST_DTYPES[info["dtype"]]).newbyteorder("<"))
        out[name] = np.array(arr).reshape(info["shape"])
    return out


def read_model_folder(folder):
    """(config dict, weights dict) of a folder with config.json + model.safetensors."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, read_safetensors(folder / "model.safetensors")


def sizes_of(cfg: dict) -> dict:
    """Sizes and constants with the reference's defaults (src/l4_gbin.c:67-81:
    kv heads default to heads, head_dim to dim/heads, eps 1e-6, theta 1e6)."""
    nh = cfg["num_attention_heads"]
    return dict(
        H=cfg["hidden_size"], I=cfg["intermediate_size"], L=cfg["num_hidden_layers"],
        nh=nh, nkv=cfg.get("num_key_value_heads", nh),
        hd=cfg.get("head_dim") or cfg["hidden_size"] // nh,
        V=cfg["vocab_size"], eps=cfg.get("rms_norm_eps", 1e-6),
        theta=cfg.get("rope_theta", 1e6), tied=bool(cfg.get("tie_word_embeddings", False)),
    )


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def embedding(table, tokens, dt):
    """x = E[token, :]  (src/l5_model.c:488-491)."""
    return table[np.asarray(tokens)].astype(dt)


def rmsnorm(x, w, eps, dt):
    """ss = sum x_j^2; inv = 1/sqrt(ss/n + eps); o_j = w_j * x_j * inv
    (src/l3_math.c:34-36,49; the weight is a plain multiplier)."""
    x = x.astype(dt)
    ss = (x * x).sum(-1, keepdims=True, dtype=dt)
    inv = dt(1) / np.sqrt(ss / dt(x.shape[-1]) + dt(eps))
    return (w.astype(dt) * x) * inv


def qk_rmsnorm(x, w, eps, dt):
    """Per head over head_dim, one weight [hd] shared by all heads, same eps as the
    layer norms (src/l3_math.c:107-114; src/l5_model.c:505-511).  x: [..., heads, hd]."""
    return rmsnorm(x, w, eps, dt)


def rope_neox(x, positions, theta, dt):
    """Half-split rotation of pairs (j, j+hd/2) with freq_j = theta^(-2j/hd),
    ang = pos*freq_j (src/l3_math.c:84-102).  x: [T, heads, hd], positions: [T].
    The reference builds freq_j by repeated f32 multiplication (:88-92); the direct
    power is used here, which agrees to rounding at the contexts tested."""
    hd = x.shape[-1]
    half = hd // 2
    freq = (np.float64(theta) ** (-2.0 * np.arange(half, dtype=np.float64) / hd)).astype(dt)
    ang = np.asarray(positions).astype(dt)[:, None] * freq[None, :]        # [T, half]
    c = np.cos(ang).astype(dt)[:, None, :]
    s = np.sin(ang).astype(dt)[:, None, :]
    a, b = x[..., :half].astype(dt), x[..., half:].astype(dt)
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def causal_attention(q, k, v, dt, window=0, scale=None):
    """scores s[h,t] = (q_h . K[t, h//group]) * scale with scale = 1/sqrt(hd), for
    t <= pos; softmax with max subtraction; o = sum p*V (src/l5_model.c:518,
    559-577; softmax src/l3_math.c:52-56).  q: [T, nh, hd]; k, v: [T, nkv, hd].
    ``window`` > 0 keeps only the keys with pos-window < t <= pos (not a feature of
    the reference; used by tests of a windowed layer)."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = dt(1) / np.sqrt(dt(hd)) if scale is None else dt(scale)
    out = np.zeros((T, nh, hd), dt)
    for pos in range(T):
        lo = 0 if window <= 0 else max(0, pos - window + 1)
        for h in range(nh):
            kh = h // group
            s = (k[lo:pos + 1, kh].astype(dt) @ q[pos, h].astype(dt)) * scale
            e = np.exp(s - s.max())
            p = e / e.sum(dtype=dt)
            out[pos, h] = p @ v[lo:pos + 1, kh].astype(dt)
    return out


def swiglu(x, wg, wu, wd, dt):
    """g = Wg x; u = Wu x; g = g/(1+exp(-g)); h = g*u; out = Wd h
    (src/l5_model.c:588-596; silu src/l3_math.c:57-62)."""
    g = x @ wg.astype(dt).T
    u = x @ wu.astype(dt).T
    g = g / (dt(1) + np.exp(-g))
    return (g * u) @ wd.astype(dt).T


def attention_block(x, W, pfx, S, positions, dt, window=0):
    """QKV projections without bias, QK-norm, then RoPE, then attention, then the
    output projection (src/l5_model.c:497-514, 580-581)."""
    T = x.shape[0]
    q = (x @ W[pfx + "q_proj.weight"].astype(dt).T).reshape(T, S["nh"], S["hd"])
    k = (x @ W[pfx + "k_proj.weight"].astype(dt).T).reshape(T, S["nkv"], S["hd"])
    v = (x @ W[pfx + "v_proj.weight"].astype(dt).T).reshape(T, S["nkv"], S["hd"])
    q = rope_neox(qk_rmsnorm(q, W[pfx + "q_norm.weight"], S["eps"], dt), positions, S["theta"], dt)
    k = rope_neox(qk_rmsnorm(k, W[pfx + "k_norm.weight"], S["eps"], dt), positions, S["theta"], dt)
    o = causal_attention(q, k, v, dt, window=window)
    return o.reshape(T, -1) @ W[pfx + "o_proj.weight"].astype(dt).T


def forward(cfg: dict, W: dict, tokens, dtype=np.float32, windows=None):
    """Logits [T, V] of one whole sequence starting at position 0
    (src/l5_model.c:461-606: pre-norm residual blocks, final norm, lm_head that
    falls back to the embedding matrix when no output matrix exists :602-604)."""
    dt = np.dtype(dtype).type
    S = sizes_of(cfg)
    T = len(tokens)
    positions = np.arange(T)
    x = embedding(W["model.embed_tokens.weight"], tokens, dt)
    for l in range(S["L"]):
        p = f"model.layers.{l}."
        h = rmsnorm(x, W[p + "input_layernorm.weight"], S["eps"], dt)
        win = 0 if windows is None else windows[l]
        x = x + attention_block(h, W, p + "self_attn.", S, positions, dt, window=win)
        h = rmsnorm(x, W[p + "post_attention_layernorm.weight"], S["eps"], dt)
        x = x + swiglu(h, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                       W[p + "mlp.down_proj.weight"], dt)
    x = rmsnorm(x, W["model.norm.weight"], S["eps"], dt)
    head = W["model.embed_tokens.weight"] if S["tied"] else W["lm_head.weight"]
    return x @ head.astype(dt).T


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------
def greedy(logits):
    """First maximum wins (strict >)  (src/l5_model.c:610-614)."""
    return int(np.argmax(logits))


def softmax32(x):
    """src/l3_math.c:52-56 in float32, sequential sum."""
    x = np.asarray(x, np.float32)
    e = np.exp(x - x.max()).astype(np.float32)
    s = np.float32(0)
    for t in e:
        s = np.float32(s + t)
    return e / s


def sample_temperature(logits, temp, r):
    """logits/=temp; softmax; first i with r <= cumsum, else n-1
    (src/l5_model.c:615-619).  ``r`` in [0,1] replaces rand()/RAND_MAX."""
    p = softmax32(np.asarray(logits, np.float32) / np.float32(temp))
    c = np.cumsum(p.astype(np.float64))
    i = int(np.searchsorted(c, r, side="left"))
    return min(i, len(p) - 1), c


def apply_repeat_penalty(logits, penalty, recent):
    """Each distinct recent id once: v>0 ? v/R : v*R  (src/main.c:204-223)."""
    out = np.array(logits, np.float32)
    if penalty == 1.0:
        return out
    seen = set()
    for i in recent:
        if 0 <= i < len(out) and i not in seen:
            seen.add(i)
            out[i] = out[i] / np.float32(penalty) if out[i] > 0 else out[i] * np.float32(penalty)
    return out


def sample_advanced(logits, temp, top_k, top_p, penalty, recent, r):
    """Repeat penalty, then greedy if temp<=0; else logits/temp, descending sort
    (ties: lower id first), keep top_k, softmax over the kept, cut at the first
    prefix whose cumsum >= top_p, renormalise, first i with r <= cumsum
    (src/main.c:225-268).  Returns (id, kept ids in order, cumulative sums)."""
    l = apply_repeat_penalty(logits, penalty, recent)
    if temp <= 0:
        return greedy(l), None, None
    l = l / np.float32(temp)
    order = np.lexsort((np.arange(len(l)), -l.astype(np.float64)))
    keep = len(l)
    if 0 < top_k < len(l):
        keep = top_k
    kept = order[:keep]
    e = np.exp((l[kept] - l[kept[0]]).astype(np.float64))
    p = e / e.sum()
    if top_p < 1.0:
        c = np.cumsum(p)
        idx = np.nonzero(c >= top_p)[0]
        last = int(idx[0]) + 1 if len(idx) else keep
        kept, p = kept[:last], p[:last]
        p = p / p.sum()
    c = np.cumsum(p)
    i = int(np.searchsorted(c, r, side="left"))
    i = min(i, len(kept) - 1)
    return int(kept[i]), kept, c
