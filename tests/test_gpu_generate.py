"""Generation through the Python entry point against the plain implementation."""
import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, model_folder, plain_logits as plain_logits_of, plain_model, random_tokens, tolerance
from plain import philox_plain, qwen3_plain as P

pytestmark = pytest.mark.gpu


def plain_generate(name, storage, prompt, n, temperature=0.0, seed=0, stream=0, stop=()):
    """Greedy or temperature generation by the plain implementation: the whole sequence
    is run again for every new token (no cache)."""
    cfg, W = plain_model(name, storage)
    toks, out = list(prompt), []
    for draw in range(n):
        logits = P.forward(cfg, W, toks, np.float32)[-1]
        if temperature <= 0:
            t = P.greedy(logits)
        else:
            t, _ = P.sample_temperature(logits, temperature, philox_plain.uniform(seed, stream, draw))
        if t in stop:
            return out, "stop"
        out.append(t)
        toks.append(t)
    return out, "length"


@pytest.fixture(scope="module")
def llms():
    from gguf2bin_b200.api import LLM
    made = {}

    def get(name, dtype, max_tokens=1024):
        key = (name, dtype, max_tokens)
        if key not in made:
            storage = "float32" if dtype == "float32" else "bfloat16"
            made[key] = LLM(model_folder(name, storage), dtype=dtype, max_tokens=max_tokens)
        return made[key]
    return get


def test_greedy_tiny_a_float32(llms):
    """Tiny A: one prompt of 7 tokens, 9 greedy steps."""
    prompt = random_tokens("a", 7, 0)
    out = llms("a", "float32").generate([prompt], n=9, temperature=0.0, top_k=0, top_p=1.0,
                                        repeat_penalty=1.0)[0]
    want, _ = plain_generate("a", "float32", prompt, 9)
    assert out.tokens == want and out.finish_reason == "length"


def test_temperature_tiny_b_unequal_batch(llms):
    """Tiny B: three unequal prompts (5, 11, 2), 6 steps at temperature 0.8, seeded.  The
    same requests alone, and in another order, draw the same tokens: a request's random
    stream is its own."""
    llm = llms("b", "float32")
    prompts = [random_tokens("b", n, 10 + i) for i, n in enumerate([5, 11, 2])]
    kw = dict(n=6, temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=1234)
    outs = llm.generate(prompts, **kw)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        want, _ = plain_generate("b", "float32", p, 6, 0.8, seed=1234, stream=i)
        assert o.tokens == want, f"request {i}"
    assert llm.generate(prompts[:1], **kw)[0].tokens == outs[0].tokens
    assert llm.generate(prompts, max_batch=1, **kw)[2].tokens == outs[2].tokens


@pytest.mark.parametrize("name,dtype", [("a", "bfloat16"), ("c", "bfloat16"), ("d", "bfloat16"), ("c", "float32")])
def test_greedy_batches_with_stop_and_reuse(llms, name, dtype):
    """Seven requests through a cache that holds three at a time; one stop token ends
    some of them early.  Greedy ids equal the plain implementation's wherever its top
    two logits are further apart than the engine's tolerance."""
    storage = "float32" if dtype == "float32" else "bfloat16"
    lens = [3, 40, 17, 1, 64 if name != "a" else 50, 9, 30]
    prompts = [random_tokens(name, n, 40 + i) for i, n in enumerate(lens)]
    n_new = 12
    ref0, _ = plain_generate(name, storage, prompts[1], n_new)
    first_seen = [j for j in range(n_new) if ref0[j] not in ref0[:j]]
    cut = first_seen[-1]      # greedy output repeats itself: stop at a token's first occurrence (may be 0)
    stop = {ref0[cut]}
    llm = llms(name, dtype, max_tokens=3 * 128)
    outs = llm.generate(prompts, n=n_new, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                        stop_ids=stop)
    cfg, W = plain_model(name, storage)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        toks = list(p)
        for j, t in enumerate(o.tokens + ([o.stop_token] if o.stop_token is not None else [])):
            logits = P.forward(cfg, W, toks, np.float32)[-1]
            top = np.sort(logits)[-2:]
            margin = 1e-4 if dtype == "float32" else 2 * tolerance(dtype, logits)
            if top[1] - top[0] > margin:
                assert t == int(np.argmax(logits)), f"request {i} token {j}"
            else:
                assert logits[t] >= top[1] - margin, f"request {i} token {j}"
            toks.append(t)
        if o.finish_reason == "stop":
            assert o.stop_token in stop and all(t not in stop for t in o.tokens)
        else:
            assert o.finish_reason == "length" and len(o.tokens) == n_new
    assert outs[1].finish_reason == "stop" and len(outs[1].tokens) == cut
    assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0


def test_filtered_sampling_is_reproducible_and_batch_independent(llms):
    llm = llms("b", "float32")
    prompts = [random_tokens("b", n, 70 + i) for i, n in enumerate([9, 4, 20, 6])]
    kw = dict(n=10, seed=99)                                  # the reference's defaults otherwise
    a = llm.generate(prompts, **kw)
    b = llm.generate(prompts, **kw)
    c = llm.generate(prompts, max_batch=3, **kw)
    assert [o.tokens for o in a] == [o.tokens for o in b] == [o.tokens for o in c]
    d = llm.generate(prompts, n=10, seed=100)
    assert [o.tokens for o in a] != [o.tokens for o in d]
    # top_k = 1 is greedy with the penalty applied, whatever the seed
    e = llm.generate(prompts[:1], n=6, top_k=1, repeat_penalty=1.0, seed=5)[0]
    assert e.tokens == plain_generate("b", "float32", prompts[0], 6)[0]


def plain_generate_filtered(name, storage, prompt, n, temp, top_k, top_p, penalty, seed, stream):
    """The reference's sampler chain (src/main.c:197-268) over the last 64 tokens of the
    prompt and what was generated so far (src/main.c:18, 327-333), by the plain implementation."""
    cfg, W = plain_model(name, storage)
    toks, out = list(prompt), []
    for draw in range(n):
        logits = P.forward(cfg, W, toks, np.float32)[-1]
        r = philox_plain.uniform(seed, stream, draw) if temp > 0 else 0.0
        t, _, _ = P.sample_advanced(logits, temp, top_k, top_p, penalty, toks[-64:], r)
        out.append(int(t))
        toks.append(int(t))
    return out


@pytest.mark.parametrize("temp,top_k", [(0.0, 0), (0.9, 1), (0.8, 5)])
def test_repeat_penalty_in_a_batch_against_plain(llms, temp, top_k):
    """A strong repeat penalty on a batch of four unequal prompts: every row must be
    penalised with its OWN recent tokens and count (a row that read another row's would
    choose other ids), and a request's tokens must not depend on its row in the batch."""
    llm = llms("b", "float32")
    prompts = [random_tokens("b", n, 90 + i) for i, n in enumerate([7, 70, 3, 21])]
    kw = dict(n=12, temperature=temp, top_k=top_k, top_p=1.0 if top_k <= 1 else 0.95,
              repeat_penalty=1.6, seed=31, ignore_eos=True)
    outs = llm.generate(prompts, **kw)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        want = plain_generate_filtered("b", "float32", p, 12, temp, top_k, kw["top_p"], 1.6, 31, i)
        assert o.tokens == want, f"request {i}"
    # the penalty must have mattered: unpenalised greedy output differs somewhere
    if temp == 0.0:
        assert any(o.tokens != plain_generate("b", "float32", p, 12)[0] for p, o in zip(prompts, outs))
    # each request in a batch of its own (row 0 every time) draws the same tokens
    one_by_one = llm.generate(prompts, max_batch=1, **kw)
    assert [o.tokens for o in one_by_one] == [o.tokens for o in outs]


@pytest.mark.parametrize("filtered", [True, False])
def test_sampling_over_a_large_vocabulary_inside_the_step(llms, filtered):
    """A vocabulary of 8,209 entries: the samplers that give a row to many blocks run inside the
    decode step and its graph (five requests in steps of eight rows, rows that start off a 16-byte
    boundary, the repeat penalty's ring).  Every token against the plain implementation."""
    llm = llms("e", "float32", max_tokens=1024)
    prompts = [random_tokens("e", n, 950 + i) for i, n in enumerate([5, 30, 2, 64, 17])]
    n_new = 12
    if filtered:
        kw = dict(temperature=0.7, top_k=40, top_p=0.9, repeat_penalty=1.3, seed=5)
        want = [plain_generate_filtered("e", "float32", p, n_new, 0.7, 40, 0.9, 1.3, 5, i) for i, p in enumerate(prompts)]
    else:
        kw = dict(temperature=0.9, top_k=0, top_p=1.0, repeat_penalty=1.0, seed=5)
        want = [plain_generate("e", "float32", p, n_new, 0.9, seed=5, stream=i)[0] for i, p in enumerate(prompts)]
    before = llm.engine.decode_graph_captures
    outs = llm.generate(prompts, n=n_new, ignore_eos=True, **kw)
    assert llm.engine.decode_graph_captures > before, "twelve steps of one shape are worth a graph"
    for i, o in enumerate(outs):
        assert o.tokens == want[i], f"request {i}"


@pytest.mark.parametrize("name", ["b", "e"])
def test_graphs_and_rows_of_padding_change_no_token_in_float32(name):
    """Sixty generation calls drawn at random (1 to 20 requests of 1 to 80 prompt tokens, 1 to 30
    new tokens, batches of 1 to 16, stop ids that end requests at any step, four ways of sampling)
    through an engine that replays graphs, fills its steps up and keeps rows of padding, and
    through one that launches every step plainly with exactly its own rows: in 32-bit arithmetic
    no row's result depends on the rows beside it, so every token and every reason to stop agrees.
    Nothing stays held in either cache."""
    from gguf2bin_b200.api import LLM
    rng = np.random.default_rng(11)
    vocab = TINY[name]["vocab_size"]
    room = TINY[name]["max_position_embeddings"] - 35
    a = LLM(model_folder(name, "float32"), dtype="float32", max_tokens=40 * 128)
    b = LLM(model_folder(name, "float32"), dtype="float32", max_tokens=40 * 128)
    b.use_graph = False
    b.engine.step_graphs = False
    ways = [dict(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0),
            dict(temperature=0.8, top_k=0, top_p=1.0, repeat_penalty=1.0),
            dict(temperature=0.7, top_k=40, top_p=0.9, repeat_penalty=1.1),
            dict(temperature=0.9, top_k=0, top_p=0.8, repeat_penalty=1.3)]
    for it in range(60):
        prompts = [rng.integers(0, vocab, int(rng.integers(1, min(81, room)))).tolist()
                   for _ in range(int(rng.integers(1, 21)))]
        kw = dict(n=int(rng.integers(1, 31)), stop_ids=rng.integers(0, vocab, int(rng.integers(0, vocab // 12))).tolist(),
                  seed=it, max_batch=int(rng.integers(1, 17)), **ways[it % 4])
        got, want = a.generate(prompts, **kw), b.generate(prompts, **kw)
        for i, (x, y) in enumerate(zip(got, want)):
            assert x.tokens == y.tokens and x.finish_reason == y.finish_reason, f"call {it}, request {i}"
        for llm in (a, b):
            assert llm.engine.cache.table.pages.n_held == 0 and llm.engine.cache.table.slots.n_held == 0
    assert a.engine.graph_captures > 10 and b.engine.graph_captures == 0


def test_rows_beyond_the_sequences_change_nothing(llms):
    """Six and eleven sequences decode as steps of eight and sixteen rows (the rows beyond them
    use the cache's spare page and slot), and keep that shape while sequences end: every
    request's tokens equal the plain implementation's, with a penalty that reads each row's own
    recent ids and a random stream per request; nothing stays held in the cache."""
    from gguf2bin_b200.engine.decode import padded_rows
    assert [padded_rows(n) for n in (1, 4, 5, 8, 9, 64, 65)] == [1, 4, 8, 8, 16, 64, 72]
    llm = llms("b", "float32", max_tokens=2048)
    eng = llm.engine
    lens = [7, 70, 3, 21, 64, 1, 33, 12, 5, 90, 2]
    prompts = [random_tokens("b", n, 300 + i) for i, n in enumerate(lens)]
    kw = dict(temperature=0.8, top_k=5, top_p=0.95, repeat_penalty=1.6, seed=77)
    want = [plain_generate_filtered("b", "float32", p, 12, 0.8, 5, 0.95, 1.6, 77, i) for i, p in enumerate(prompts)]
    # stop ids that end some requests early, at different steps
    stops = {want[1][4], want[4][8], want[9][2]}
    for n_req in (6, 11):
        shapes_before = set(eng.decode_runners)
        outs = llm.generate(prompts[:n_req], n=12, stop_ids=stops, **kw)
        for i, o in enumerate(outs):
            cut = next((j for j, t in enumerate(want[i]) if t in stops), 12)
            assert o.tokens == want[i][:cut], f"{n_req} requests, request {i}"
        assert any(len(o.tokens) < 12 for o in outs)
        new_shapes = set(eng.decode_runners) - shapes_before
        assert all(k[0] in (1, 2, 3, 4, 8, 16) for k in new_shapes) and any(k[0] == padded_rows(n_req) for k in new_shapes)
        assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


def test_context_limit_and_errors(llms):
    from gguf2bin_b200.engine import GenerationError, StepEntry, StepError
    llm = llms("a", "float32")
    p = random_tokens("a", 60, 5)
    out = llm.generate([p], n=20, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)[0]
    assert out.finish_reason == "context" and len(out.tokens) == 4       # 64 positions in all
    assert out.tokens == plain_generate("a", "float32", p, 4)[0]
    out = llm.generate([p], n=20, ctx=62, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0)[0]
    assert out.finish_reason == "context" and len(out.tokens) == 2
    with pytest.raises(GenerationError, match="context"):
        llm.generate([random_tokens("a", 65, 6)], n=1)
    held = llm.engine.cache.table.pages.n_held
    seq = llm.open_sequence()
    for bad in ([StepEntry(seq, [300], [0])], [StepEntry(seq, [], [])], [StepEntry(seq, [1, 2], [2])],
                [StepEntry(seq, [1] * 65, [])], [StepEntry(seq, [1], []), StepEntry(seq, [2], [])]):
        with pytest.raises(StepError):
            llm.step(bad)
        assert seq.length == 0 and llm.engine.cache.table.pages.n_held == held
    llm.close_sequence(seq)
    with pytest.raises(StepError, match="not live"):
        llm.step([StepEntry(seq, [1], [0])])


def test_step_launched_ahead_is_taken_back(llms):
    """The decode session launches each next step before the host has seen the last tokens.
    Here the caller then feeds other tokens than the sampled ones (and later ends one sequence
    early): the step launched ahead must leave no trace, neither in the cache nor in the draw
    counters of the seeded sampler.  Temperature 0.7, two sequences, against the plain
    implementation fed the same tokens."""
    from gguf2bin_b200.engine.backend import EngineBackend
    from gguf2bin_b200.sampling import SamplingParams
    llm = llms("b", "float32")
    temp, seed = 0.7, 77
    backend = EngineBackend(llm.engine, SamplingParams.plain(temp), seed, max_context=256)
    prompts = [random_tokens("b", 6, 31), random_tokens("b", 9, 32)]
    handles = [backend.open(i, 64) for i in range(2)]
    cfg, W = plain_model("b", "float32")
    fed = [list(p) for p in prompts]
    draws = [0, 0]

    def plain_next(i):
        logits = P.forward(cfg, W, fed[i], np.float32)[-1]
        t, _ = P.sample_temperature(logits, temp, philox_plain.uniform(seed, i, draws[i]))
        draws[i] += 1
        return t

    got = backend.prefill(handles, prompts)
    assert got == [plain_next(0), plain_next(1)]
    live = [0, 1]
    for step in range(8):
        if step == 3:                              # the caller overrides the sampled tokens
            got = [(t + 1) % cfg["vocab_size"] for t in got]
        if step == 6:                              # sequence 0 ends; the batch changes
            backend.close(handles[0])
            live, got = [1], got[1:]
        for i, t in zip(live, got):
            fed[i].append(t)
        got = backend.decode([handles[i] for i in live], got)
        assert got == [plain_next(i) for i in live], f"step {step}"
    backend.close(handles[1])


@pytest.mark.parametrize("filtered", [False, True])
def test_rows_of_sequences_that_end_go_on_as_padding(llms, filtered):
    """Eight sequences, then seven, six and five, in steps of eight rows.  Sequences end in the middle of the batch while a
    step is launched ahead; the others keep their rows and that step.  Right after one of them
    ended the caller feeds other tokens than the sampled ones, so the step launched ahead is
    taken back from rows of which one has just become padding (not with the repeat penalty,
    whose recent ids on the device are the sampled ones).  Every token against the plain
    implementation fed the same tokens, with each request's own random stream and recent ids."""
    from gguf2bin_b200.engine.backend import EngineBackend
    from gguf2bin_b200.sampling import SamplingParams
    llm = llms("b", "float32", max_tokens=2048)
    eng = llm.engine
    temp, seed = 0.7, 123
    params = SamplingParams(temperature=temp, top_k=6, top_p=0.9, repeat_penalty=1.5) if filtered \
        else SamplingParams.plain(temp)
    backend = EngineBackend(eng, params, seed, max_context=256)
    prompts = [random_tokens("b", n, 400 + n) for n in (6, 9, 63, 2, 30, 64, 11, 17)]
    handles = [backend.open(i, 100) for i in range(8)]
    cfg, W = plain_model("b", "float32")
    fed = [list(p) for p in prompts]
    draws = [0] * 8

    def plain_next(i):
        logits = P.forward(cfg, W, fed[i], np.float32)[-1]
        r = philox_plain.uniform(seed, i, draws[i])
        draws[i] += 1
        if filtered:
            return int(P.sample_advanced(logits, temp, 6, 0.9, 1.5, fed[i][-64:], r)[0])
        return P.sample_temperature(logits, temp, r)[0]

    got = backend.prefill(handles, prompts)
    assert got == [plain_next(i) for i in range(8)]
    live = list(range(8))
    ends = {2: 3, 4: 0, 5: 6}                          # step -> the sequence that ends before it
    session = None
    for step in range(9):
        if step in ends:
            k = live.index(ends[step])
            backend.close(handles[ends[step]])
            live, got = live[:k] + live[k + 1:], got[:k] + got[k + 1:]
            if step > 2:
                assert backend._session is session, "the batch was put together anew"
        if step in (4, 7) and not filtered:            # the caller overrides the sampled tokens (the recent
            got = [(t + 1 + i) % cfg["vocab_size"] for i, t in enumerate(got)]     # ids on the device are the sampled ones)
        for i, t in zip(live, got):
            fed[i].append(t)
        got = backend.decode([handles[i] for i in live], got)
        session = backend._session
        assert session.runner.batch == 8
        assert got == [plain_next(i) for i in live], f"step {step}"
    assert session.rows == [1, 2, 4, 5, 7]
    for i in live:
        backend.close(handles[i])
    backend.finish()
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0


def test_decode_graphs_are_kept_by_shape_not_by_call(llms):
    """A decode graph belongs to the engine and to a shape (sequences, page-table width,
    sampling): a second call with the same shape captures nothing, and a batch of 64 whose
    sequences end one per step passes through eight shapes of rows, not 63, and captures a graph
    for each at most.  Tokens are compared with an engine that never uses graphs."""
    from gguf2bin_b200.engine.backend import EngineBackend
    from gguf2bin_b200.sampling import SamplingParams
    llm = llms("c", "bfloat16", max_tokens=64 * 128)
    eng = llm.engine
    prompts = [random_tokens("c", 5 + (i % 7), 500 + i) for i in range(8)]
    kw = dict(n=14, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    first = llm.generate(prompts, **kw)
    after_first = eng.decode_graph_captures
    assert after_first >= 1, "fourteen steps of one shape are worth a graph"
    again = llm.generate(prompts, **kw)
    assert eng.decode_graph_captures == after_first, "the same shape in a later call captured a graph again"
    assert [o.tokens for o in again] == [o.tokens for o in first]
    llm.use_graph = False
    try:
        plain = llm.generate(prompts, **kw)
    finally:
        llm.use_graph = True
    assert [o.tokens for o in plain] == [o.tokens for o in first]

    backend = EngineBackend(eng, SamplingParams.plain(0.0), seed=0, max_context=128)
    many = [random_tokens("c", 3 + (i % 5), 600 + i) for i in range(64)]
    handles = [backend.open(i, 100) for i in range(64)]
    got = backend.prefill(handles, many)
    before = eng.decode_graph_captures
    live = list(range(64))
    while len(live) > 1:
        backend.close(handles[live[0]])
        live, got = live[1:], got[1:]
        got = backend.decode([handles[i] for i in live], got)
    backend.close(handles[live[0]])
    backend.finish()
    captured = eng.decode_graph_captures - before
    assert captured <= 8, f"{captured} graphs for a shrinking batch"
    assert eng.cache.table.slots.n_held == 0 and eng.cache.table.pages.n_held == 0


def test_graphs_that_are_let_go_do_not_spoil_a_capture(llms):
    """Shapes come and go (sequences that end at different steps, more shapes than the engine
    keeps runners for), and Python's collector of cycles is set to run at every few allocations:
    a graph that is released while another is being captured would end that capture with an
    error.  Tokens equal those of an engine that uses no graphs."""
    import gc
    llm = llms("c", "bfloat16", max_tokens=32 * 128)
    eng = llm.engine
    prompts = [random_tokens("c", 3 + (i % 6), 800 + i) for i in range(28)]
    kw = dict(temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    sizes = (12, 20, 3, 9, 28, 5, 20)                 # steps of 16, 24, 3, 16, 32, 8 and 24 rows
    kept, eng.DECODE_RUNNERS_KEPT = eng.DECODE_RUNNERS_KEPT, 2
    thresholds = gc.get_threshold()
    before = eng.decode_graph_captures
    try:
        gc.set_threshold(5, 1, 1)
        with_graphs = [llm.generate(prompts[:b], n=8, max_batch=b, **kw) for b in sizes]
    finally:
        gc.set_threshold(*thresholds)
        eng.DECODE_RUNNERS_KEPT = kept
    assert eng.decode_graph_captures - before >= 6
    llm.use_graph = False
    try:
        plain = [llm.generate(prompts[:b], n=8, max_batch=b, **kw) for b in sizes]
    finally:
        llm.use_graph = True
    assert [[o.tokens for o in call] for call in with_graphs] == [[o.tokens for o in call] for call in plain]


def test_the_cycle_collector_rests_while_a_graph_is_captured():
    """Releasing a CUDA graph is forbidden while a stream captures, and Python's collector of
    cycles may release one at any allocation: ``capture_graph`` holds it off and puts it back."""
    import gc
    from gguf2bin_b200.engine.step import capture_graph
    x = torch.zeros(4, device="cuda")
    seen = []

    def launch():
        seen.append(gc.isenabled())
        x.add_(1.0)
        return "result"
    assert gc.isenabled()
    graph, result = capture_graph(launch)
    assert seen == [False] and gc.isenabled() and result == "result"
    graph.replay()
    graph.replay()
    assert x.tolist() == [2.0] * 4
    gc.disable()
    try:
        capture_graph(launch)
        assert not gc.isenabled(), "a collector that was off stays off"
    finally:
        gc.enable()


@pytest.mark.parametrize("use_graph", [False, True])
def test_steps_taken_back_at_page_edges_leave_the_same_bits(llms, use_graph):
    """Every step is followed by a step launched ahead that is then taken back, with sequences
    whose positions cross a page edge meanwhile (the decode attention fetches old pages early,
    on a hint of the position that a take-back moves down by one): the logits of every real
    step equal, bit for bit, those of a session that never ran ahead."""
    from gguf2bin_b200.engine import DecodeSession, StepEntry
    from gguf2bin_b200.sampling import Sampler, SamplingParams
    llm = llms("d", "bfloat16", max_tokens=1024)
    eng = llm.engine
    prompts = [random_tokens("d", n, 700 + n) for n in (61, 126, 190)]
    fed = [random_tokens("d", 8, 900 + i) for i in range(3)]

    def run(ahead: bool):
        seqs = [eng.open_sequence() for _ in prompts]
        for s, p in zip(seqs, prompts):
            eng.cache.reserve(s, len(p) + 12)
        eng.step([StepEntry(s, p, ()) for s, p in zip(seqs, prompts)])
        session = DecodeSession(eng, seqs, Sampler(eng.cache.seq_state, eng.device), SamplingParams.plain(0.0),
                                use_graph=use_graph, eager_steps=1)
        out = []
        for i in range(8):
            session.set_tokens([f[i] for f in fed])
            session.run()
            out.append(session.logits.clone())
            if ahead:                                  # a step nobody asked for, and its undoing
                session.run()
                session._ahead = session.read_tokens()
                session.take_back()
        lengths = [s.length for s in seqs]
        for s in seqs:
            eng.close_sequence(s)
        return out, lengths

    plain, n0 = run(False)
    with_ahead, n1 = run(True)
    assert n0 == n1 == [len(p) + 8 for p in prompts]
    for i, (a, b) in enumerate(zip(plain, with_ahead)):
        assert torch.equal(a, b), f"step {i}"
    # and they are the plain implementation's logits
    ref = plain_logits_of("d", "bfloat16", prompts[1] + fed[1])
    assert_close(np.stack([x[1].cpu().numpy() for x in plain]), ref[len(prompts[1]):], "bfloat16", "sequence 1")
