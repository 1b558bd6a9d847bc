"""Places where a cache or a batch goes wrong first: long decoding, the first tokens of a
sequence, a far key among hundreds, page boundaries, a slot used again; and the trace
replay program run as a user runs it."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, model_folder, plain_logits, plain_model, random_tokens
from plain import qwen3_plain as P

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def make_engine(name, dtype, max_tokens=1024):
    from gguf2bin_b200.engine import Engine, Model
    storage = "float32" if dtype == "float32" else "bfloat16"
    return Engine(Model.from_folder(model_folder(name, storage), dtype=dtype), max_tokens=max_tokens)


@pytest.mark.parametrize("name,dtype", [("c", "float32"), ("c", "bfloat16"), ("d", "bfloat16")])
def test_long_decoding(name, dtype):
    """A short prompt, then some three hundred tokens one by one across several pages."""
    from gguf2bin_b200.engine import StepEntry
    n = 330 if name == "c" else 300
    toks = random_tokens(name, n, 21)
    eng = make_engine(name, dtype)
    seq = eng.open_sequence()
    got = [eng.step([StepEntry(seq, toks[:5], range(5))]).cpu().numpy()]
    for t in toks[5:]:
        got.append(eng.step([StepEntry(seq, [t], [0])]).cpu().numpy())
    storage = "float32" if dtype == "float32" else "bfloat16"
    assert_close(np.concatenate(got), plain_logits(name, storage, toks), dtype, f"{name}/{dtype} long decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_every_cut(dtype):
    """The first six tokens of a sequence, cut into steps in every possible way."""
    from gguf2bin_b200.engine import StepEntry
    storage = "float32" if dtype == "float32" else "bfloat16"
    toks = random_tokens("b", 6, 3)
    ref = plain_logits("b", storage, toks)
    eng = make_engine("b", dtype)
    for mask in range(32):                               # a cut after token i where bit i is set
        cuts = [i + 1 for i in range(5) if mask >> i & 1] + [6]
        seq, got, a = eng.open_sequence(), [], 0
        for b in cuts:
            got.append(eng.step([StepEntry(seq, toks[a:b], range(b - a))]).cpu().numpy())
            a = b
        eng.close_sequence(seq)
        assert_close(np.concatenate(got), ref, dtype, f"cuts {cuts}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_stands_out(dtype):
    """Weights made so that one key, hundreds of positions back, takes nearly all the
    attention of the last query: with queries and keys that ignore their input except
    for a marker token, a cache that drops, shifts or mixes up one position shows at
    once.  Checked against the plain implementation on the same weights."""
    from gguf2bin_b200.engine import Engine, Model, StepEntry
    from gguf2bin_b200.weights import write_random_model, write_safetensors
    from helpers import tmp_root
    name, storage = "c", ("float32" if dtype == "float32" else "bfloat16")
    cfg, W = plain_model(name, storage)
    W = {k: v.copy() for k, v in W.items()}
    A, B, hd = 7, 8, TINY[name]["head_dim"]
    # token A's embedding is direction 0, which only layer 0's queries read; token B's is
    # direction 1, which only its keys and values read; both land in the two slowest
    # rotary dimensions of every head, so the match survives hundreds of positions
    E = W["model.embed_tokens.weight"]
    E[A] = 0
    E[A, 0] = 4.0
    E[B] = 0
    E[B, 1] = 4.0
    for p, n_heads, col in (("q_proj", TINY[name]["num_attention_heads"], 0),
                            ("k_proj", TINY[name]["num_key_value_heads"], 1)):
        w = W[f"model.layers.0.self_attn.{p}.weight"]
        w[:, 0] = 0
        w[:, 1] = 0
        for h in range(n_heads):
            w[h * hd + hd // 2 - 1, col] = 1.5
            w[h * hd + hd - 1, col] = 1.5
    W["model.layers.0.self_attn.v_proj.weight"][:, 1] = 0.5
    folder = tmp_root() / f"far_key_{storage}"
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(TINY[name]))
    tdt = torch.float32 if storage == "float32" else torch.bfloat16
    write_safetensors(folder / "model.safetensors",
                      [(k, v.shape, tdt, (lambda v=v: torch.from_numpy(v).to(tdt))) for k, v in W.items()])
    cfg2, W2 = P.read_model_folder(folder)
    toks = [t if t not in (A, B) else 9 for t in random_tokens(name, 400, 9)]
    toks[37] = B                                         # the far key
    toks[-1] = A                                         # the query that looks for it
    ref = P.forward(cfg2, W2, toks, np.float32)
    base = P.forward(cfg2, W2, toks[:37] + [10] + toks[38:], np.float32)
    from helpers import tolerance
    tol = tolerance(dtype, ref)
    assert np.abs(ref[-1] - base[-1]).max() > 3 * tol, \
        "the construction does not make the far key matter"
    eng = Engine(Model.from_folder(folder, dtype=dtype), max_tokens=1024)
    seq = eng.open_sequence()
    got = [eng.step([StepEntry(seq, toks[:300], range(300))]).cpu().numpy()]
    for t in toks[300:]:
        got.append(eng.step([StepEntry(seq, [t], [0])]).cpu().numpy())
    assert_close(np.concatenate(got), ref, dtype, "far key")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_page_edges_and_slot_reuse(dtype):
    """Prompts that end just before, at and just after a page boundary, decoded across
    it, on a cache whose only free pages are the ones the previous sequence left full
    of other data."""
    from gguf2bin_b200.engine import StepEntry
    storage = "float32" if dtype == "float32" else "bfloat16"
    eng = make_engine("c", dtype, max_tokens=192)        # three pages: one sequence at a time
    for i, plen in enumerate([63, 64, 65, 127, 128, 129]):
        toks = random_tokens("c", plen + 4, 50 + i)
        seq = eng.open_sequence()
        got = [eng.step([StepEntry(seq, toks[:plen], [plen - 1])]).cpu().numpy()]
        for t in toks[plen:]:
            got.append(eng.step([StepEntry(seq, [t], [0])]).cpu().numpy())
        eng.close_sequence(seq)
        ref = plain_logits("c", storage, toks)[plen - 1:]
        assert_close(np.concatenate(got), ref, dtype, f"prompt of {plen}")


@pytest.mark.parametrize("name,dtype", [("b", "float32"), ("b", "bfloat16"), ("d", "float32"), ("d", "bfloat16")])
def test_mixed_steps(name, dtype):
    """Steps whose sequences are at different stages: while X decodes one token, Y brings a
    whole prompt of 70 tokens and Z continues a prompt that was cut at a page edge (64 tokens
    in, 30 more now); then X and Y decode while Z brings its last piece.  Logits of every
    place against the plain implementation of each sequence whole."""
    from gguf2bin_b200.engine import StepEntry
    storage = "float32" if dtype == "float32" else "bfloat16"
    X, Y, Z = random_tokens(name, 24, 61), random_tokens(name, 73, 62), random_tokens(name, 99, 63)
    eng = make_engine(name, dtype)
    sx, sy, sz = (eng.open_sequence() for _ in range(3))
    got = {"x": [], "y": [], "z": []}

    def run(parts):
        """parts: (key, sequence, tokens); every place is wanted."""
        out = eng.step([StepEntry(s, t, range(len(t))) for _, s, t in parts]).cpu().numpy()
        o = 0
        for key, _, t in parts:
            got[key].append(out[o:o + len(t)])
            o += len(t)

    run([("x", sx, X[:20]), ("z", sz, Z[:64])])                         # two prompts, Z's cut at the page edge
    run([("x", sx, X[20:21]), ("y", sy, Y[:70]), ("z", sz, Z[64:94])])  # decode + fresh prompt + continuation
    run([("z", sz, Z[94:99]), ("x", sx, X[21:22]), ("y", sy, Y[70:71])])
    run([("y", sy, Y[71:72]), ("x", sx, X[22:23])])
    run([("x", sx, X[23:24]), ("y", sy, Y[72:73])])
    for key, toks in (("x", X), ("y", Y), ("z", Z)):
        assert_close(np.concatenate(got[key]), plain_logits(name, storage, toks), dtype,
                     f"{name}/{dtype} sequence {key}")
    for s in (sx, sy, sz):
        eng.close_sequence(s)


def test_padding_rows_change_nothing():
    """A batch with a one-token neighbour gives bit-equal logits to the same request
    alone: rows of padding (the step is filled up to 64 rows: 14 of them alone, 13 with
    the neighbour) and rows of other sequences change no bit, no reduction spans rows."""
    from gguf2bin_b200.engine import StepEntry
    for dtype in ("float32", "bfloat16"):
        eng = make_engine("b", dtype)
        toks, other = random_tokens("b", 50, 1), random_tokens("b", 1, 2)
        s = eng.open_sequence()
        alone = eng.step([StepEntry(s, toks, range(50))]).clone()
        eng.close_sequence(s)
        s1, s2 = eng.open_sequence(), eng.open_sequence()
        both = eng.step([StepEntry(s2, other, [0]), StepEntry(s1, toks, range(50))])
        assert torch.equal(both[1:], alone)
        eng.close_sequence(s1); eng.close_sequence(s2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """bin/trace_run as a user runs it: a batch of unequal requests, shorter ones ending
    earlier, then a second batch in the freed slots, with some steps wanting nothing."""
    storage = "float32" if dtype == "float32" else "bfloat16"
    reqs = {"r0": random_tokens("b", 40, 80), "r1": random_tokens("b", 9, 81),
            "r2": random_tokens("b", 70, 82), "r3": random_tokens("b", 33, 83)}
    steps, expect = [], {}
    n = 0
    for batch in (["r0", "r1"], ["r2", "r3"]):
        heads = {r: max(1, len(reqs[r]) - 6) for r in batch}
        done = dict(heads)
        entries = [{"id": r, "tokens": reqs[r][:heads[r]], "want": [0, heads[r] - 1]} for r in batch]
        expect[n] = [(r, i) for r in batch for i in (0, heads[r] - 1)]
        steps.append({"step": n, "entries": entries, "end": [r for r in batch if done[r] == len(reqs[r])]})
        n += 1
        live = [r for r in batch if done[r] < len(reqs[r])]
        while live:
            want_now = n % 2 == 0
            entries = [{"id": r, "tokens": [reqs[r][done[r]]], "want": [0] if want_now else []} for r in live]
            if want_now:
                expect[n] = [(r, done[r]) for r in live]
            for r in live:
                done[r] += 1
            ended = [r for r in live if done[r] == len(reqs[r])]
            steps.append({"step": n, "entries": entries, "end": ended})
            live = [r for r in live if r not in ended]
            n += 1
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model",
                           str(model_folder("b", storage)), "--dtype", dtype, "--out", str(out),
                           "--max-tokens", "192"],
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True,
                          capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    V = TINY["b"]["vocab_size"]
    for s in steps:
        f = out / f"{s['step']}.f32"
        if s["step"] not in expect:
            assert not f.exists()
            continue
        got = np.fromfile(f, "<f4").reshape(-1, V)
        ref = np.stack([plain_logits("b", storage, reqs[r])[i] for r, i in expect[s["step"]]])
        assert_close(got, ref, dtype, f"trace step {s['step']}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_shape_that_comes_back_is_replayed_from_a_graph(dtype):
    """Steps of one shape (two prompts of 70 and 40 tokens, logits wanted at three places):
    the first two run plainly, the third is captured in a CUDA graph, later ones replay it.
    Every run has other tokens, other slots and other pages, and each is compared with the
    plain implementation; the same tokens again give the same bits as the plain run did."""
    from gguf2bin_b200.engine import StepEntry
    name = "c"
    eng = make_engine(name, dtype, max_tokens=2048)
    assert eng.step_graphs, "the library's own parts declare themselves fit for graphs"
    storage = "float32" if dtype == "float32" else "bfloat16"
    hold = [eng.open_sequence() for _ in range(3)]          # so that later runs get other slots and pages
    first = None
    for run in range(5):
        seed = 300 if run == 4 else 300 + run               # the last run repeats the first one's tokens
        a, b = random_tokens(name, 70, seed), random_tokens(name, 40, seed + 50)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        got = eng.step([StepEntry(sa, a, (0, 69)), StepEntry(sb, b, (39,))]).cpu().numpy()
        want = np.stack([plain_logits(name, storage, a)[0], plain_logits(name, storage, a)[69],
                         plain_logits(name, storage, b)[39]])
        assert_close(got, want, dtype, f"run {run}")
        if run == 0:
            first = got
        if run == 4:
            assert np.array_equal(got, first), "a replayed step differs from the plain run of the same tokens"
        if run % 2 == 0:                                     # keep some, close some: the free pages change
            eng.close_sequence(sa)
            eng.close_sequence(sb)
        else:
            eng.close_sequence(hold.pop())
    assert len(eng._graphs) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prompts_of_other_lengths_find_a_graph(dtype):
    """Prompt steps are filled up to a multiple of 64 rows with a padding sequence on the cache's
    spare page, so prompts of 129 to 192 tokens are one shape: the first two run plainly, the third
    is captured, the others replay that graph, each with its own length, tokens, slot and pages and
    each against the plain implementation at three places.  The same for two prompts in one step
    whose lengths change while their sum's bucket and their tiles do not.  A length of exactly 192
    needs no padding and is a shape of its own.  Nothing is held by the padding."""
    from gguf2bin_b200.engine import StepEntry
    name = "c"
    eng = make_engine(name, dtype, max_tokens=4096)
    storage = "float32" if dtype == "float32" else "bfloat16"
    def prompt_graphs():
        return sum(1 for key in eng._graphs if key[0] == "prompt")
    for i, n in enumerate((150, 129, 191, 170, 135)):
        toks = random_tokens(name, n, 400 + i)
        s = eng.open_sequence()
        places = (0, n // 2, n - 1)
        got = eng.step([StepEntry(s, toks, places)]).cpu().numpy()
        assert_close(got, plain_logits(name, storage, toks)[list(places)], dtype, f"prompt of {n}")
        # and it decodes on from there: the padding left nothing in its pages
        nxt = random_tokens(name, 1, 450 + i)
        got = eng.step([StepEntry(s, nxt, [0])]).cpu().numpy()
        assert_close(got, plain_logits(name, storage, toks + nxt)[-1:], dtype, f"token after a prompt of {n}")
        if i % 2:
            eng.close_sequence(s)
    assert prompt_graphs() == 1, "five lengths of one bucket: one graph"
    for i, (na, nb) in enumerate(((100, 60), (110, 50), (127, 40), (90, 64))):     # 154 to 167 rows, three tiles of 64 rows and two of 128
        a, b = random_tokens(name, na, 500 + i), random_tokens(name, nb, 550 + i)
        sa, sb = eng.open_sequence(), eng.open_sequence()
        got = eng.step([StepEntry(sa, a, (na - 1,)), StepEntry(sb, b, (0, nb - 1))]).cpu().numpy()
        want = np.stack([plain_logits(name, storage, a)[-1], plain_logits(name, storage, b)[0],
                         plain_logits(name, storage, b)[-1]])
        assert_close(got, want, dtype, f"prompts of {na} and {nb}")
        eng.close_sequence(sa)
        eng.close_sequence(sb)
    assert prompt_graphs() == 2
    toks = random_tokens(name, 192, 600)
    s = eng.open_sequence()
    assert_close(eng.step([StepEntry(s, toks, range(192))]).cpu().numpy(), plain_logits(name, storage, toks), dtype,
                 "prompt of 192")
    eng.close_sequence(s)
    assert prompt_graphs() == 2, "a shape seen once is not captured"


@pytest.mark.parametrize("name,dtype,seed", [("b", "float32", 1), ("c", "bfloat16", 2), ("d", "bfloat16", 3), ("d", "float32", 4)])
def test_random_schedules(name, dtype, seed):
    """A seeded random walk over what a caller may do: sequences open at any time, bring their
    next one to forty tokens in steps shared with whoever else is ready (prompts, continuations
    and single tokens mixed), want logits at random places, and close when done, in a cache with
    room for about half of them, so that pages and slots are reused all the time.  Every logit
    that was asked for equals the plain implementation's at that position of that sequence."""
    from gguf2bin_b200.engine import StepEntry
    storage = "float32" if dtype == "float32" else "bfloat16"
    rng = np.random.default_rng(seed)
    limit = min(TINY[name]["max_position_embeddings"], 200)
    eng = make_engine(name, dtype, max_tokens=64 * 10)
    pending = [random_tokens(name, int(rng.integers(1, limit)), 4000 + 10 * seed + i) for i in range(14)]
    live = []                                     # [sequence, tokens, fed so far, wanted: list of (position, row of logits)]
    checked = 0
    while pending or live:
        # open what fits
        while pending and len(live) < 5:
            need = -(-len(pending[0]) // 64)
            if need > eng.cache.table.pages.n_free - sum(-(-len(t) // 64) - len(s.pages) for s, t, _, _ in live):
                break
            live.append([eng.open_sequence(), pending.pop(0), 0, []])
        assert live, "the cache is too small for the longest request"
        # a step over a random non-empty subset of the live sequences
        chosen = [x for x in live if rng.random() < 0.7] or [live[int(rng.integers(len(live)))]]
        entries, asked = [], []
        for x in chosen:
            seq, toks, fed, _ = x
            n = int(min(len(toks) - fed, rng.choice([1, 1, 2, 7, 40])))
            want = sorted(set(int(w) for w in rng.integers(0, n, int(rng.integers(0, 3)))))
            entries.append(StepEntry(seq, toks[fed:fed + n], want))
            asked.append((x, fed, n, want))
        out = eng.step(entries)
        rows = out.cpu().numpy() if out is not None else np.zeros((0, 0))
        r = 0
        for x, fed, n, want in asked:
            for w in want:
                x[3].append((fed + w, rows[r]))
                r += 1
            x[2] = fed + n
        assert r == len(rows)
        for x in [x for x in live if x[2] == len(x[1])]:
            seq, toks, _, wanted = x
            if wanted:
                ref = plain_logits(name, storage, toks)
                assert_close(np.stack([row for _, row in wanted]), ref[[p for p, _ in wanted]], dtype,
                             f"{name}/{dtype} sequence of {len(toks)} tokens")
                checked += len(wanted)
            eng.close_sequence(seq)
            live.remove(x)
    assert checked > 20
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


def test_a_context_of_33000_tokens_cut_three_ways():
    """Far beyond what the plain implementation can follow in the tests' time, so the engine is
    compared with itself (the kernels' own long-context tests compare with the plain attention):
    a prompt of 33,000 tokens whole in one step; in pieces of 8,192; and with its last three
    tokens decoded one by one.  The logits at the last four places and at two places in the
    middle agree within the bfloat16 bound."""
    from gguf2bin_b200.engine import Engine, Model, StepEntry
    from helpers import tmp_root
    from gguf2bin_b200.weights import write_random_model
    cfg = dict(TINY["d"], max_position_embeddings=40960)
    folder = write_random_model(tmp_root() / "tiny_d_long", cfg, 5, "bfloat16")
    eng = Engine(Model.from_folder(folder, dtype="bfloat16"), max_tokens=33024 + 64)
    n = 33000
    toks = np.random.default_rng(11).integers(0, cfg["vocab_size"], n).tolist()
    places = [8191, 16400, n - 4, n - 3, n - 2, n - 1]

    s = eng.open_sequence()
    whole = eng.step([StepEntry(s, toks, places)]).cpu().numpy()
    eng.close_sequence(s)

    s = eng.open_sequence()
    got = []
    for a in range(0, n, 8192):
        b = min(n, a + 8192)
        want = [p - a for p in places if a <= p < b]
        out = eng.step([StepEntry(s, toks[a:b], want)])
        if want:
            got.append(out.cpu().numpy())
    eng.close_sequence(s)
    pieces = np.concatenate(got)

    s = eng.open_sequence()
    got = [eng.step([StepEntry(s, toks[:n - 3], [8191, 16400, n - 4])]).cpu().numpy()]
    for t in toks[n - 3:]:
        got.append(eng.step([StepEntry(s, [t], [0])]).cpu().numpy())
    eng.close_sequence(s)
    decoded = np.concatenate(got)

    assert np.isfinite(whole).all() and np.abs(whole).max() > 0.1
    assert_close(pieces, whole, "bfloat16", "pieces of 8,192 against the whole prompt")
    assert_close(decoded, whole, "bfloat16", "last three tokens decoded against the whole prompt")
    assert eng.cache.table.pages.n_held == 0
