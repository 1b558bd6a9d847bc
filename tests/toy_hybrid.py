"""A whole toy architecture defined OUTSIDE the package, as a plug-in module: its own
config.json keys, its own tensor names, a mixer with a fixed-size state beside attention
layers, an embedding with a multiplier, and a plain numpy forward pass for the tests.

Importing the module registers everything (``register_architecture``, ``register_mixer``,
``register_embedding``); with ``GGUF2BIN_B200_PLUGINS=toy_hybrid`` and this folder on
PYTHONPATH the command line and ``bin/trace_run`` know the architecture too.  It is no model
of anyone's: it exists to show that another architecture needs no change to the package.
"""
import numpy as np
import torch

from gguf2bin_b200.cache import StateNeed
from gguf2bin_b200.config import (ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                                  register_architecture)
from gguf2bin_b200.parts import register_embedding, register_mixer
from gguf2bin_b200.weights import Expected

ARCHITECTURE = "ToyHybridForCausalLM"


class LeakyStateMixer:
    """s_t = a * s_{t-1} + (1 - a) * (W_in h_t), out_t = W_out (s_t * tanh(s_t)); a per channel in
    (0, 1).  Its only memory is s, of fixed size per sequence."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.width = int(spec["width"])

    @classmethod
    def expected(cls, spec, hidden_size):
        w = spec["width"]
        return {"mix.w_in": Expected((w, hidden_size)), "mix.w_out": Expected((hidden_size, w)),
                "mix.leak": Expected((w,), init="scale")}

    def bind(self, tensors):
        self.w_in, self.w_out = tensors["mix.w_in"].float(), tensors["mix.w_out"].float()
        self.a = torch.sigmoid(tensors["mix.leak"].float())

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def forward(self, h, ctx, view, residual32):
        u = h.float() @ self.w_in.T
        t0 = 0
        for slot, n in zip(ctx.slots, ctx.q_lens):
            s, outs = view.states[slot], []
            for t in range(t0, t0 + n):
                s = self.a * s + (1 - self.a) * u[t]
                outs.append(s * torch.tanh(s))
            view.states[slot] = s
            residual32[t0:t0 + n] += torch.stack(outs) @ self.w_out.T
            t0 += n


class MultipliedEmbedding:
    def __init__(self, spec, vocab_size, hidden_size, dtype, device):
        self.name, self.multiplier = spec["name"], float(spec["multiplier"])

    @classmethod
    def expected(cls, spec, vocab_size, hidden_size):
        return {spec["name"]: Expected((vocab_size, hidden_size))}

    def bind(self, tensors):
        self.table = tensors[self.name].contiguous()

    def forward(self, tok_ids, out32, ctx):
        from gguf2bin_b200 import kernels
        kernels.embed_rows(self.table, tok_ids, out32)
        out32.mul_(self.multiplier)


def read_config(d) -> ModelSpec:
    """config.json of this architecture: d_model, n_layer, pattern ("A" attention / "S" state, one
    letter per layer), heads, kv_heads, head_size, state_width, ffn, vocab, ctx, eps, theta,
    emb_multiplier, eos."""
    try:
        pattern = str(d["pattern"])
        if len(pattern) != int(d["n_layer"]) or set(pattern) - {"A", "S"}:
            raise ConfigError("config.json: pattern needs one letter, A or S, per layer")
        eps = float(d["eps"])
        norm = PartSpec.make("rmsnorm", eps=eps)
        attention = PartSpec.make(
            "gqa_attention", n_heads=int(d["heads"]), n_kv_heads=int(d["kv_heads"]), head_dim=int(d["head_size"]),
            qk_norm=PartSpec.make("rmsnorm", eps=eps),
            position=PartSpec.make("rope_neox", theta=float(d["theta"]), rotary_dim=int(d["head_size"])),
            window=0, scale=None,
            names=(("q", "att.q"), ("k", "att.k"), ("v", "att.v"), ("o", "att.o"), ("q_norm", "att.qn"),
                   ("k_norm", "att.kn")))
        state = PartSpec.make("toy_leaky_state", width=int(d["state_width"]))
        ffn = PartSpec.make("swiglu", intermediate_size=int(d["ffn"]),
                            names=(("gate", "ffn.g"), ("up", "ffn.u"), ("down", "ffn.d")))
        block = PartSpec.make("prenorm", names=(("mixer_norm", "ln1"), ("ffn_norm", "ln2")))
        layers = tuple(LayerSpec(block=block, mixer=attention if c == "A" else state, feed_forward=ffn,
                                 norm=norm, prefix=f"blocks.{i}.") for i, c in enumerate(pattern))
        eos = d.get("eos")
        return ModelSpec(
            architecture=ARCHITECTURE, hidden_size=int(d["d_model"]), vocab_size=int(d["vocab"]),
            max_positions=int(d["ctx"]), layers=layers,
            schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
            embedding=PartSpec.make("toy_multiplied_embedding", name="wte", multiplier=float(d["emb_multiplier"])),
            final_norm=PartSpec.make("rmsnorm", eps=eps, name="ln_f"),
            head=PartSpec.make("lm_head", tied=True, name="unused_head"),
            stop_token_ids=() if eos is None else (int(eos),), source=dict(d))
    except KeyError as e:
        raise ConfigError(f"config.json: missing required key {e.args[0]!r}") from None


register_mixer("toy_leaky_state", LeakyStateMixer)
register_embedding("toy_multiplied_embedding", MultipliedEmbedding)
register_architecture(ARCHITECTURE, read_config)

CONFIG = dict(architectures=[ARCHITECTURE], d_model=80, n_layer=3, pattern="ASA", heads=4, kv_heads=2,
              head_size=32, state_width=24, ffn=136, vocab=173, ctx=256, eps=1e-5, theta=5e4,
              emb_multiplier=4.0, eos=None)


def plain_forward(cfg, W, tokens):
    """Logits of every position, whole sequence, no cache, from the plain parts."""
    from plain import qwen3_plain as P
    f = np.float32
    T, eps = len(tokens), cfg["eps"]
    positions = np.arange(T)
    nh, nkv, hd = cfg["heads"], cfg["kv_heads"], cfg["head_size"]
    x = P.embedding(W["wte"], tokens, f) * f(cfg["emb_multiplier"])
    for i, c in enumerate(cfg["pattern"]):
        pfx = f"blocks.{i}."
        h = P.rmsnorm(x, W[pfx + "ln1"], eps, f)
        if c == "A":
            q = P.qk_rmsnorm((h @ W[pfx + "att.q"].T).reshape(T, nh, hd), W[pfx + "att.qn"], eps, f)
            k = P.qk_rmsnorm((h @ W[pfx + "att.k"].T).reshape(T, nkv, hd), W[pfx + "att.kn"], eps, f)
            v = (h @ W[pfx + "att.v"].T).reshape(T, nkv, hd)
            q, k = P.rope_neox(q, positions, cfg["theta"], f), P.rope_neox(k, positions, cfg["theta"], f)
            x = x + P.causal_attention(q, k, v, f).reshape(T, -1) @ W[pfx + "att.o"].T
        else:
            a = 1 / (1 + np.exp(-W[pfx + "mix.leak"]))
            u = h @ W[pfx + "mix.w_in"].T
            s, outs = np.zeros_like(u[0]), []
            for t in range(T):
                s = a * s + (1 - a) * u[t]
                outs.append(s * np.tanh(s))
            x = x + np.stack(outs) @ W[pfx + "mix.w_out"].T
        h = P.rmsnorm(x, W[pfx + "ln2"], eps, f)
        x = x + P.swiglu(h, W[pfx + "ffn.g"], W[pfx + "ffn.u"], W[pfx + "ffn.d"], f)
    return P.rmsnorm(x, W["ln_f"], eps, f) @ W["wte"].T
