"""The parts, alone and in arrangements the Qwen3 configuration never asks for: each part
against the plain implementation's function; a model whose layers differ (a windowed
mixer beside full ones, so two cache groups; a layer run twice; a layer that reads
another layer's keys and values; no position encoding); and toy parts defined here — a
mixer with a state of its own, a feed-forward with routing, another position encoding —
registered, built and stepped without a change to the framework's files."""
import math

import numpy as np
import pytest
import torch

from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def gpu(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(DEV)


# ---------------------------------------------------------------------------
# building models from specs, with random tensors, and a plain forward over specs
# ---------------------------------------------------------------------------
def attention_spec(nh, nkv, hd, eps, theta=None, window=0, shared_kv=False, position=None):
    from gguf2bin_b200.config import PartSpec
    if position is None:
        position = (PartSpec.make("rope_neox", theta=theta, rotary_dim=hd) if theta
                    else PartSpec.make("none"))
    return PartSpec.make(
        "gqa_attention", n_heads=nh, n_kv_heads=nkv, head_dim=hd,
        qk_norm=PartSpec.make("rmsnorm", eps=eps), position=position, window=window, scale=None,
        shared_kv=shared_kv,
        names=(("q", "attn.q.weight"), ("k", "attn.k.weight"), ("v", "attn.v.weight"),
               ("o", "attn.o.weight"), ("q_norm", "attn.qn.weight"), ("k_norm", "attn.kn.weight")))


def swiglu_spec(inter):
    from gguf2bin_b200.config import PartSpec
    return PartSpec.make("swiglu", intermediate_size=inter,
                         names=(("gate", "ffn.gate.weight"), ("up", "ffn.up.weight"),
                                ("down", "ffn.down.weight")))


def make_spec(hidden, vocab, mixers, ffns, eps, schedule=None, tied=True, embedding=None, head=None):
    from gguf2bin_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    norm = PartSpec.make("rmsnorm", eps=eps)
    block = PartSpec.make("prenorm", names=(("mixer_norm", "n1.weight"), ("ffn_norm", "n2.weight")))
    layers = tuple(LayerSpec(block=block, mixer=m, feed_forward=f, norm=norm, prefix=f"L{i}.")
                   for i, (m, f) in enumerate(zip(mixers, ffns)))
    schedule = schedule or [(i, None) for i in range(len(layers))]
    return ModelSpec(architecture="TestModel", hidden_size=hidden, vocab_size=vocab, max_positions=512,
                     layers=layers, schedule=tuple(ScheduleEntry(a, b) for a, b in schedule),
                     embedding=embedding or PartSpec.make("token_embedding", name="emb.weight"),
                     final_norm=PartSpec.make("rmsnorm", eps=eps, name="norm.weight"),
                     head=head or PartSpec.make("lm_head", tied=tied, name="head.weight"))


def build(spec, dtype, seed=0):
    """(engine, weights as float32 numpy by name); bfloat16 runs get weights that are
    already bfloat16 values, so both sides compute from the same numbers."""
    from gguf2bin_b200.engine import Engine, Model, expected_tensors
    from gguf2bin_b200.weights import random_tensor
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = {n: random_tensor(e, seed, i, tdt, 0.05, 0.1)
               for i, (n, e) in enumerate(expected_tensors(spec).items()) if not e.optional}
    model = Model(spec, dtype=dtype)
    model.bind({n: t.to(DEV) for n, t in tensors.items()})
    return Engine(model, max_tokens=2048), {n: t.float().numpy() for n, t in tensors.items()}


def plain_attention(x, W, pfx, m, positions, kv_store, layer, cache_layer, eps):
    """One attention mixer by the plain functions; ``kv_store`` keeps each storage
    layer's whole-sequence k and v so that a shared_kv layer can read them."""
    nh, nkv, hd = m["n_heads"], m["n_kv_heads"], m["head_dim"]
    T = x.shape[0]
    pos = m["position"]

    def encode(a):
        if pos.kind == "rope_neox":
            return P.rope_neox(a, positions, pos["theta"], np.float32)
        if pos.kind == "toy_xpos":
            return toy_position_plain(a, positions, pos["rate"])
        return a
    q = (x @ W[pfx + "attn.q.weight"].T).reshape(T, nh, hd)
    q = encode(P.qk_rmsnorm(q, W[pfx + "attn.qn.weight"], eps, np.float32))
    if not m.get("shared_kv"):
        k = (x @ W[pfx + "attn.k.weight"].T).reshape(T, nkv, hd)
        k = encode(P.qk_rmsnorm(k, W[pfx + "attn.kn.weight"], eps, np.float32))
        v = (x @ W[pfx + "attn.v.weight"].T).reshape(T, nkv, hd)
        kv_store[cache_layer] = (k, v)
    k, v = kv_store[cache_layer]
    o = P.causal_attention(q, k, v, np.float32, window=m["window"])
    return o.reshape(T, -1) @ W[pfx + "attn.o.weight"].T


def plain_forward(spec, W, tokens, eps, toy_mixers=None):
    x = P.embedding(W["emb.weight"], tokens, np.float32) * np.float32(spec.embedding.get("multiplier", 1.0))
    positions = np.arange(len(tokens))
    kv_store = {}
    for position, e in enumerate(spec.schedule):
        layer = spec.layers[e.layer]
        pfx = layer.prefix
        h = P.rmsnorm(x, W[pfx + "n1.weight"], eps, np.float32)
        if layer.mixer.kind == "gqa_attention":
            x = x + plain_attention(h, W, pfx, layer.mixer, positions, kv_store, e.layer,
                                    spec.cache_owner(position), eps)
        else:
            x = x + toy_mixers[layer.mixer.kind](h, W, pfx)
        h = P.rmsnorm(x, W[pfx + "n2.weight"], eps, np.float32)
        if layer.feed_forward.kind == "swiglu":
            x = x + P.swiglu(h, W[pfx + "ffn.gate.weight"], W[pfx + "ffn.up.weight"],
                             W[pfx + "ffn.down.weight"], np.float32)
        else:
            x = x + toy_mixers[layer.feed_forward.kind](h, W, pfx)
    x = P.rmsnorm(x, W["norm.weight"], eps, np.float32)
    logits = x @ (W["emb.weight"] if spec.head["tied"] else W["head.weight"]).T
    if spec.head.get("cap"):                       # the toy head: scaled, then capped smoothly
        logits = np.float32(spec.head["cap"]) * np.tanh(logits * np.float32(spec.head["scale"] / spec.head["cap"]))
    return logits


def run_cuttings(eng, requests):
    """Logits of every position of every request, three ways: whole and alone; a prompt
    then single tokens; all requests as one unequal batch followed by single tokens."""
    from gguf2bin_b200.engine import StepEntry
    ways = {"whole": [], "stepwise": [], "batched": []}
    for toks in requests:
        s = eng.open_sequence()
        ways["whole"].append(eng.step([StepEntry(s, toks, range(len(toks)))]).cpu().numpy())
        eng.close_sequence(s)
        s = eng.open_sequence()
        head = max(1, len(toks) // 2)
        got = [eng.step([StepEntry(s, toks[:head], range(head))]).cpu().numpy()]
        for t in toks[head:]:
            got.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy())
        eng.close_sequence(s)
        ways["stepwise"].append(np.concatenate(got))
    seqs = [eng.open_sequence() for _ in requests]
    heads = [max(1, len(t) - 5) for t in requests]
    out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(seqs, requests, heads)]).cpu().numpy()
    got, o = [], 0
    for h in heads:
        got.append([out[o:o + h]])
        o += h
    done = list(heads)
    live = [j for j in range(len(requests)) if done[j] < len(requests[j])]
    while live:
        out = eng.step([StepEntry(seqs[j], [requests[j][done[j]]], [0]) for j in live]).cpu().numpy()
        for r, j in enumerate(live):
            got[j].append(out[r:r + 1])
            done[j] += 1
        live = [j for j in live if done[j] < len(requests[j])]
    for s in seqs:
        eng.close_sequence(s)
    ways["batched"] = [np.concatenate(g) for g in got]
    return ways


def check(eng, spec, W, requests, dtype, eps, toy=None):
    from helpers import assert_close
    ways = run_cuttings(eng, requests)
    for i, toks in enumerate(requests):
        ref = plain_forward(spec, W, toks, eps, toy)
        for way, outs in ways.items():
            assert_close(outs[i], ref, dtype, f"request {i} {way}")
    assert eng.cache.table.pages.n_held == 0


def some_requests(vocab, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


# ---------------------------------------------------------------------------
# each part of the library alone
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from gguf2bin_b200.config import PartSpec
    from gguf2bin_b200.parts import norm_class
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    spec = PartSpec.make("rmsnorm", eps=3e-5)
    norm = norm_class(spec)(spec, 100, tdt, DEV)
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((9, 100)).astype(np.float32), (1 + 0.1 * rng.standard_normal(100)).astype(np.float32)
    norm.bind(gpu(w))
    out = torch.empty(9, 100, dtype=tdt, device=DEV)
    norm.forward(gpu(x), out)
    ref = P.rmsnorm(x, w, 3e-5, np.float32)
    tol = 2e-6 if dtype == "float32" else 2.0 ** -8
    np.testing.assert_allclose(out.float().cpu().numpy(), ref, rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_part(dtype):
    """Widths that are and are not multiples of eight (fused gate/up row order)."""
    from gguf2bin_b200.engine.workspace import Workspace
    from gguf2bin_b200.parts import feed_forward_class
    from gguf2bin_b200.parts.base import StepContext
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    for inter in (40, 100):
        spec = swiglu_spec(inter)
        ffn = feed_forward_class(spec)(spec, 72, tdt, DEV)
        rng = np.random.default_rng(inter)
        W = {n: (0.1 * rng.standard_normal(s)).astype(np.float32) for n, s in
             (("ffn.gate.weight", (inter, 72)), ("ffn.up.weight", (inter, 72)), ("ffn.down.weight", (72, inter)))}
        W = {n: gpu(w, tdt).float().cpu().numpy() for n, w in W.items()}
        ffn.bind({n: gpu(w, tdt) for n, w in W.items()})
        h = gpu(rng.standard_normal((7, 72)).astype(np.float32), tdt)
        res = torch.zeros(7, 72, device=DEV)
        ctx = StepContext(7, 1, None, None, None, None, 64, Workspace(DEV), tdt)
        ffn.forward(h, ctx, res)
        ref = P.swiglu(h.float().cpu().numpy(), W["ffn.gate.weight"], W["ffn.up.weight"], W["ffn.down.weight"], np.float32)
        tol = 1e-5 if dtype == "float32" else 2.0 ** -7
        assert np.abs(res.cpu().numpy() - ref).max() <= tol * max(1, np.abs(ref).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_position_part(dtype):
    """The rotary table of the position part drives the fused kernel; partial rotation
    leaves the tail of each head untouched."""
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.config import PartSpec
    from gguf2bin_b200.parts import position_class
    tdt = torch.float32 if dtype == "float32" else torch.bfloat16
    hd, rot, nh = 48, 32, 3
    spec = PartSpec.make("rope_neox", theta=777.0, rotary_dim=rot)
    pos = position_class(spec)(spec, hd, DEV)
    inv_freq, r = pos.fused_rotation()
    assert r == rot
    rng = np.random.default_rng(1)
    positions = [0, 1, 5, 300]
    q = gpu(rng.standard_normal((4, nh * hd)).astype(np.float32), tdt)
    out = torch.empty_like(q)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    rope = torch.empty(4, r // 2, 2, device=DEV)
    kernels.rope_table(pos_t, inv_freq, rope)
    kernels.qknorm_rope_cache(q, nh, 0, hd, None, None, 0.0, rope, r, pos_t,
                              torch.zeros(4, dtype=torch.int32, device=DEV), None, None, 64, out)
    x = q.float().cpu().numpy().reshape(4, nh, hd)
    ref = np.concatenate([P.rope_neox(x[..., :rot], positions, 777.0, np.float32), x[..., rot:]], -1)
    tol = 3e-6 if dtype == "float32" else 2.0 ** -8
    np.testing.assert_allclose(out.float().cpu().numpy().reshape(4, nh, hd), ref, rtol=tol, atol=tol)
    # the part run as a step of its own (what a mixer that does not fuse it calls): q and k in place
    from gguf2bin_b200.engine.workspace import Workspace
    from gguf2bin_b200.parts.base import StepContext
    k = gpu(rng.standard_normal((4, 2 * hd)).astype(np.float32), tdt)
    kx = k.float().cpu().numpy().reshape(4, 2, hd)
    q2 = q.clone()
    ctx = StepContext(4, 1, None, pos_t, torch.zeros(4, dtype=torch.int32, device=DEV), None, 64,
                      Workspace(DEV), tdt)
    pos.apply(q2, k, ctx)
    kref = np.concatenate([P.rope_neox(kx[..., :rot], positions, 777.0, np.float32), kx[..., rot:]], -1)
    np.testing.assert_allclose(q2.float().cpu().numpy().reshape(4, nh, hd), ref, rtol=tol, atol=tol)
    np.testing.assert_allclose(k.float().cpu().numpy().reshape(4, 2, hd), kref, rtol=tol, atol=tol)


# ---------------------------------------------------------------------------
# arrangements beyond the architecture
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_that_differ(dtype):
    """Layer 0 full attention with 4/2 heads of 16; layer 1 a window of 11 with 2/1 heads
    of 32 and no position encoding; layer 2 full again; feed-forwards of different widths.
    Two kinds of need, three cache groups."""
    eps = 1e-5
    mixers = [attention_spec(4, 2, 16, eps, theta=1e4), attention_spec(2, 1, 32, eps, window=11),
              attention_spec(4, 2, 16, eps, theta=1e4)]
    spec = make_spec(48, 97, mixers, [swiglu_spec(64), swiglu_spec(20), swiglu_spec(36)], eps)
    eng, W = build(spec, dtype)
    assert len(eng.cache.groups) == 2
    keys = sorted(eng.cache.groups)
    assert [len(eng.cache.groups[k]["layers"]) for k in keys] in ([1, 2], [2, 1])
    check(eng, spec, W, some_requests(97, [70, 9, 130, 23]), dtype, eps)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_is_data(dtype):
    """Layer 0 runs twice, each run with a cache of its own; layer 2 has no k/v of its
    own and reads the keys and values that layer 1 stored at schedule position 0."""
    eps = 1e-6
    mixers = [attention_spec(3, 1, 16, eps, theta=1e4), attention_spec(4, 2, 16, eps, theta=5e3),
              attention_spec(6, 2, 16, eps, theta=5e3, shared_kv=True)]
    spec = make_spec(40, 61, mixers, [swiglu_spec(24)] * 3, eps,
                     schedule=[(1, None), (2, 0), (0, None), (0, None)], tied=False)
    eng, W = build(spec, dtype, seed=3)
    assert "L2.attn.k.weight" not in W and eng.model.cache_needs()[1] is None
    check(eng, spec, W, some_requests(61, [66, 5, 20]), dtype, eps)


# ---------------------------------------------------------------------------
# toy parts, defined here, registered from here
# ---------------------------------------------------------------------------
class DecayMixer:
    """s_t = a * s_{t-1} + W_in h_t (per channel, a in (0,1)); out_t = W_out s_t.  Its
    only memory is the state s of fixed size per sequence: no keys, no pages."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.width = int(spec["width"])
        self.hidden, self.dtype = hidden_size, dtype

    @classmethod
    def expected(cls, spec, hidden_size):
        from gguf2bin_b200.weights import Expected
        w = spec["width"]
        return {"mix.in.weight": Expected((w, hidden_size)), "mix.out.weight": Expected((hidden_size, w)),
                "mix.decay.weight": Expected((w,), init="scale")}

    def bind(self, tensors):
        self.w_in = tensors["mix.in.weight"].float()
        self.w_out = tensors["mix.out.weight"].float()
        self.decay = torch.sigmoid(tensors["mix.decay.weight"].float())

    def cache_need(self):
        from gguf2bin_b200.cache import StateNeed
        return StateNeed((self.width,), torch.float32)

    def forward(self, h, ctx, view, residual32):
        u = h.float() @ self.w_in.T
        t0 = 0
        for slot, n in zip(ctx.slots, ctx.q_lens):
            s = view.states[slot]
            outs = []
            for t in range(t0, t0 + n):
                s = self.decay * s + u[t]
                outs.append(s)
            view.states[slot] = s
            residual32[t0:t0 + n] += torch.stack(outs) @ self.w_out.T
            t0 += n


def decay_mixer_plain(h, W, pfx):
    a = 1 / (1 + np.exp(-W[pfx + "mix.decay.weight"]))
    u = h @ W[pfx + "mix.in.weight"].T
    s, out = np.zeros_like(u[0]), []
    for t in range(len(u)):
        s = a * s + u[t]
        out.append(s)
    return np.stack(out) @ W[pfx + "mix.out.weight"].T


class RoutedFeedForward:
    """Two experts, each a single matrix pair; every token goes to the expert whose
    router logit (float32) is larger, weighted by the softmax of the two."""

    def __init__(self, spec, hidden_size, dtype, device):
        self.inter = int(spec["intermediate_size"])

    @classmethod
    def expected(cls, spec, hidden_size):
        from gguf2bin_b200.weights import Expected
        i = spec["intermediate_size"]
        return {"moe.router.weight": Expected((2, hidden_size)), "moe.up.weight": Expected((2 * i, hidden_size)),
                "moe.down.weight": Expected((2 * hidden_size, i))}

    def bind(self, tensors):
        self.router = tensors["moe.router.weight"].float()
        self.up = tensors["moe.up.weight"].float().view(2, self.inter, -1)
        self.down = tensors["moe.down.weight"].float().view(2, -1, self.inter)

    def forward(self, h, ctx, residual32):
        x = h.float()
        logits = x @ self.router.T
        p = torch.softmax(logits, -1)
        choice = logits.argmax(-1)
        for e in range(2):
            rows = (choice == e).nonzero().flatten()
            if len(rows):
                y = torch.relu(x[rows] @ self.up[e].T) @ self.down[e].T
                residual32[rows] += p[rows, e:e + 1] * y


def routed_plain(h, W, pfx):
    logits = h @ W[pfx + "moe.router.weight"].T
    e = np.exp(logits - logits.max(-1, keepdims=True))
    p = e / e.sum(-1, keepdims=True)
    inter = W[pfx + "moe.up.weight"].shape[0] // 2
    out = np.zeros_like(h)
    for t in range(len(h)):
        c = int(np.argmax(logits[t]))
        up = W[pfx + "moe.up.weight"][c * inter:(c + 1) * inter]
        down = W[pfx + "moe.down.weight"].reshape(2, -1, inter)[c]
        out[t] = p[t, c] * (np.maximum(h[t] @ up.T, 0) @ down.T)
    return out


class ToyPosition:
    """Not a rotation: scales dimension j of q and k by exp(-rate * pos * j / hd) and
    exp(+...) would be xpos; here both get (1 + rate * pos)^(-j/hd), which cannot be
    expressed by the fused rotary table, so the mixer must take its unfused path."""

    def __init__(self, spec, head_dim, device):
        self.rate, self.hd = float(spec["rate"]), head_dim
        self.expo = -(torch.arange(head_dim, dtype=torch.float32, device=device) / head_dim)

    def fused_rotation(self):
        return None

    def apply(self, q, k, ctx):
        base = (1 + self.rate * ctx.tok_pos.float())[:, None]
        f = base ** self.expo[None, :]                              # [T, hd]
        for a in (q, k):
            v = a.view(a.shape[0], -1, self.hd)
            v.copy_((v.float() * f[:, None, :]).to(a.dtype))


def toy_position_plain(a, positions, rate):
    hd = a.shape[-1]
    base = (1 + np.float32(rate) * np.asarray(positions, np.float32))[:, None]
    f = base ** (-(np.arange(hd, dtype=np.float32) / hd))[None, :]
    return a * f[:, None, :]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_parts_register_build_and_step(dtype):
    from gguf2bin_b200.cache import StateView
    from gguf2bin_b200.config import PartSpec
    from gguf2bin_b200.parts import register_feed_forward, register_mixer, register_position
    register_mixer("toy_decay", DecayMixer)
    register_feed_forward("toy_routed", RoutedFeedForward)
    register_position("toy_xpos", ToyPosition)
    eps = 1e-5
    mixers = [attention_spec(4, 2, 16, eps, position=PartSpec.make("toy_xpos", rate=0.05)),
              PartSpec.make("toy_decay", width=24),
              attention_spec(2, 2, 32, eps, theta=1e4)]
    # a routing decision flips on a rounding difference, so the routed feed-forward is
    # compared in float32 only
    routed = PartSpec.make("toy_routed", intermediate_size=16) if dtype == "float32" else swiglu_spec(24)
    ffns = [swiglu_spec(40), routed, swiglu_spec(40)]
    spec = make_spec(32, 83, mixers, ffns, eps)
    eng, W = build(spec, dtype, seed=7)
    assert isinstance(eng.cache.view(1), StateView) and tuple(eng.cache.view(1).states.shape[1:]) == (24,)
    toy = {"toy_decay": decay_mixer_plain, "toy_routed": routed_plain}
    check(eng, spec, W, some_requests(83, [40, 3, 90, 17]), dtype, eps, toy)
    # a reused slot starts from a cleared state: run the same requests again
    check(eng, spec, W, some_requests(83, [40, 3, 90, 17]), dtype, eps, toy)


def test_generation_with_a_state_mixer():
    """The decay mixer's state cannot be rewound, so the decode session must not run a step
    ahead of the caller for this model: three sequences decode together, the caller overrides
    the sampled tokens once, and the sequences end at different steps (each end starts a new
    session for those that are left).  Every token equals the plain implementation's greedy
    choice over the tokens fed so far; a state that had taken a token twice would not."""
    from gguf2bin_b200.config import PartSpec
    from gguf2bin_b200.engine.backend import EngineBackend
    from gguf2bin_b200.parts import register_mixer
    from gguf2bin_b200.sampling import SamplingParams
    register_mixer("toy_decay", DecayMixer)
    eps = 1e-5
    mixers = [attention_spec(4, 2, 16, eps, theta=1e4), PartSpec.make("toy_decay", width=24)]
    spec = make_spec(32, 83, mixers, [swiglu_spec(40), swiglu_spec(24)], eps)
    eng, W = build(spec, "float32", seed=11)
    toy = {"toy_decay": decay_mixer_plain}
    backend = EngineBackend(eng, SamplingParams.plain(0.0), seed=0, max_context=256)
    prompts = some_requests(83, [9, 4, 17], seed=5)
    handles = [backend.open(i, 64) for i in range(3)]
    fed = [list(p) for p in prompts]

    def plain_next(i):
        return int(np.argmax(plain_forward(spec, W, fed[i], eps, toy)[-1]))

    got = backend.prefill(handles, prompts)
    assert got == [plain_next(i) for i in range(3)]
    live = [0, 1, 2]
    for step in range(10):
        if step == 3:                              # the caller feeds other tokens than the sampled ones
            got = [(t + 7) % 83 for t in got]
        if step in (5, 7):                         # a sequence ends; the others go on as a new batch
            gone = live[0]
            backend.close(handles[gone])
            live, got = live[1:], got[1:]
        for i, t in zip(live, got):
            fed[i].append(t)
        got = backend.decode([handles[i] for i in live], got)
        assert got == [plain_next(i) for i in live], f"step {step}"
    backend.close(handles[live[0]])
    backend.finish()
    assert eng.cache.table.slots.n_held == 0


class ScaledEmbedding:
    """Toy end: the table's row times a constant."""

    def __init__(self, spec, vocab_size, hidden_size, dtype, device):
        self.name, self.multiplier = spec["name"], float(spec["multiplier"])

    @classmethod
    def expected(cls, spec, vocab_size, hidden_size):
        from gguf2bin_b200.weights import Expected
        return {spec["name"]: Expected((vocab_size, hidden_size))}

    def bind(self, tensors):
        self.table = tensors[self.name].contiguous()

    def forward(self, tok_ids, out32, ctx):
        from gguf2bin_b200 import kernels
        kernels.embed_rows(self.table, tok_ids, out32)
        out32.mul_(self.multiplier)


class CappedHead:
    """Toy end: logits = cap * tanh(scale * (h . E^T) / cap) over the embedding's table."""

    def __init__(self, spec, vocab_size, hidden_size, dtype, device):
        self.scale, self.cap = float(spec["scale"]), float(spec["cap"])

    @classmethod
    def expected(cls, spec, vocab_size, hidden_size):
        return {}

    def bind(self, tensors, embedding):
        self.matrix = embedding.table

    def forward(self, h, logits32, ctx):
        from gguf2bin_b200 import kernels
        kernels.linear(h, self.matrix, logits32)
        logits32.copy_(self.cap * torch.tanh(logits32 * (self.scale / self.cap)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_ends_register_build_and_step(dtype):
    """Another architecture's embedding (scaled) and head (a scale and a smooth cap on the
    logits, tied to the embedding) are parts like the others: registered from here, chosen by
    the spec, and the model only walks them."""
    from gguf2bin_b200.config import PartSpec
    from gguf2bin_b200.parts import register_embedding, register_head
    register_embedding("toy_scaled_embedding", ScaledEmbedding)
    register_head("toy_capped_head", CappedHead)
    eps = 1e-6
    spec = make_spec(48, 97, [attention_spec(3, 1, 16, eps, theta=1e4)] * 2, [swiglu_spec(40)] * 2, eps,
                     embedding=PartSpec.make("toy_scaled_embedding", name="emb.weight", multiplier=6.5),
                     head=PartSpec.make("toy_capped_head", tied=True, name="unused", scale=9.0, cap=1.5))
    eng, W = build(spec, dtype, seed=13)
    assert not eng.model.graph_safe          # the toy ends do not say they are fit for graphs
    assert "unused" not in W
    check(eng, spec, W, some_requests(97, [33, 2, 70]), dtype, eps)
