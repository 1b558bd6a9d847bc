#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ from the reference's own C code.

What it does (CPU only, no network):
  1. builds deterministic tiny weights for two Qwen3 configurations (``CASES``);
  2. writes them as a G2BX file whose slots are all F32 (header layout:
     include/g2b.h:51-56, src/l5_model.c:286-302; roles include/g2b.h:19-23);
  3. compiles src/l1..l6 of the reference with ``driver.c`` (scalar build: no
     -mavx2, because the AVX2 rmsnorm of src/l3_math.c:25-31 drops elements when
     n % 32 is in [8,31]);
  4. feeds the token ids one by one through ``model_forward`` (src/l5_model.c:461)
     and stores the logits of every position as ``<case>_logits.npy``.

Usage:  python tests/golden/make_golden.py <checkout of AnonymoDGH/gguf2bin>
The test ``tests/test_plain_vs_golden.py`` rebuilds the same weights with
``case_weights`` and compares the plain implementation with the stored logits.
"""
from __future__ import annotations

import struct
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent

CASES = {
    # name: (config.json-style dict, seed, number of tokens fed)
    "tiny_a": (dict(architectures=["Qwen3ForCausalLM"], hidden_size=64, intermediate_size=128,
                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                    vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                    tie_word_embeddings=True, max_position_embeddings=64), 0, 16),
    "tiny_b": (dict(architectures=["Qwen3ForCausalLM"], hidden_size=96, intermediate_size=224,
                    num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
                    vocab_size=311, rope_theta=1e6, rms_norm_eps=1e-5,
                    tie_word_embeddings=False, max_position_embeddings=128), 1, 17),
}


def _splitmix64(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def det_normal(seed: int, stream: int, n: int) -> np.ndarray:
    """n standard normals that depend only on (seed, stream, index): a counter hash
    (splitmix64) turned into normals by Box-Muller in float64."""
    with np.errstate(over="ignore"):
        idx = np.arange(n, dtype=np.uint64)
        key = _splitmix64(np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream))
        a = _splitmix64(key ^ (idx * np.uint64(2)))
        b = _splitmix64(key ^ (idx * np.uint64(2) + np.uint64(1)))
    u1 = ((a >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (b >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    return np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def tensor_names(cfg: dict) -> list[tuple[str, tuple, bool]]:
    """(safetensors name, shape, is_norm) in a fixed order."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd, V = (cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                      cfg["vocab_size"])
    out = [("model.embed_tokens.weight", (V, H), False), ("model.norm.weight", (H,), True)]
    if not cfg["tie_word_embeddings"]:
        out.append(("lm_head.weight", (V, H), False))
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        out += [(p + "input_layernorm.weight", (H,), True),
                (p + "self_attn.q_proj.weight", (nh * hd, H), False),
                (p + "self_attn.k_proj.weight", (nkv * hd, H), False),
                (p + "self_attn.v_proj.weight", (nkv * hd, H), False),
                (p + "self_attn.o_proj.weight", (H, nh * hd), False),
                (p + "self_attn.q_norm.weight", (hd,), True),
                (p + "self_attn.k_norm.weight", (hd,), True),
                (p + "post_attention_layernorm.weight", (H,), True),
                (p + "mlp.gate_proj.weight", (I, H), False),
                (p + "mlp.up_proj.weight", (I, H), False),
                (p + "mlp.down_proj.weight", (H, I), False)]
    return out


def case_weights(name: str) -> tuple[dict, dict, list[int]]:
    """(config, weights by safetensors name as float32, token ids) of a case:
    matrices N(0, 0.02), norm weights 1 + N(0, 0.1)."""
    cfg, seed, n_tok = CASES[name]
    W = {}
    for i, (tname, shape, is_norm) in enumerate(tensor_names(cfg)):
        z = det_normal(seed, i, int(np.prod(shape))).reshape(shape)
        W[tname] = ((1.0 + 0.1 * z) if is_norm else 0.02 * z).astype(np.float32)
    ids = (_splitmix64(np.arange(n_tok, dtype=np.uint64) + np.uint64(1000 + seed))
           % np.uint64(cfg["vocab_size"])).astype(np.int64).tolist()
    return cfg, W, ids


# role numbers of include/g2b.h:19-23
_ROLE = {"model.embed_tokens.weight": 0, "model.norm.weight": 1, "lm_head.weight": 2,
         "input_layernorm.weight": 3, "self_attn.q_proj.weight": 4, "self_attn.k_proj.weight": 5,
         "self_attn.v_proj.weight": 6, "self_attn.o_proj.weight": 7, "self_attn.q_norm.weight": 8,
         "self_attn.k_norm.weight": 9, "post_attention_layernorm.weight": 10,
         "mlp.gate_proj.weight": 11, "mlp.up_proj.weight": 12, "mlp.down_proj.weight": 13}


def write_g2bx_f32(path: Path, cfg: dict, W: dict) -> None:
    slots, blobs, off = b"", [], 0
    for name, arr in W.items():
        if name.startswith("model.layers."):
            _, _, layer, rest = name.split(".", 3)
            role, layer = _ROLE[rest], int(layer)
        else:
            role, layer = _ROLE[name], 0xFFFF
        raw = np.ascontiguousarray(arr, np.float32).tobytes()
        slots += struct.pack("<BHBIQ", role, layer, 0, len(raw), off)   # type 0 = T_F32
        blobs.append((off, raw))
        off = (off + len(raw) + 63) & ~63
    flags = 2 | (1 if cfg["tie_word_embeddings"] else 0)               # F_QK_NORM | F_TIE_EMBD
    with open(path, "wb") as f:
        f.write(b"G2BX" + struct.pack("<HBB", 1, 2, flags))           # ver 1, ARCH_QWEN3
        f.write(struct.pack("<8i2f", cfg["hidden_size"], cfg["intermediate_size"],
                            cfg["num_hidden_layers"], cfg["num_attention_heads"],
                            cfg["num_key_value_heads"], cfg["vocab_size"],
                            cfg["max_position_embeddings"], cfg["head_dim"],
                            cfg["rms_norm_eps"], cfg["rope_theta"]))
        f.write(struct.pack("<I", len(W)) + slots)
        pos = 0
        for o, raw in blobs:
            f.write(b"\0" * (o - pos))
            f.write(raw)
            pos = o + len(raw)
        f.write(b"\0" * (off - pos))


def main() -> int:
    if len(sys.argv) < 2:
        print("usage: make_golden.py <checkout of AnonymoDGH/gguf2bin>", file=sys.stderr)
        return 2
    ref = Path(sys.argv[1])
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        exe = tmp / "dump_logits"
        srcs = [str(ref / "src" / f"l{i}_{n}.c") for i, n in
                [(1, "gguf"), (2, "codec"), (3, "math"), (4, "gbin"), (5, "model"), (6, "token")]]
        subprocess.run(["gcc", "-O2", "-std=gnu99", f"-I{ref / 'include'}", "-w",
                        str(HERE / "driver.c"), *srcs, "-lm", "-o", str(exe)], check=True)
        for name in CASES:
            cfg, W, ids = case_weights(name)
            g2bx, out = tmp / f"{name}.g2bx", tmp / f"{name}.bin"
            write_g2bx_f32(g2bx, cfg, W)
            subprocess.run([str(exe), str(g2bx), str(out), ",".join(map(str, ids))], check=True,
                           stderr=subprocess.DEVNULL)
            logits = np.fromfile(out, np.float32).reshape(len(ids), cfg["vocab_size"])
            np.save(HERE / f"{name}_logits.npy", logits)
            print(name, logits.shape, "abs max %.4f" % np.abs(logits).max())
    return 0


if __name__ == "__main__":
    sys.exit(main())
