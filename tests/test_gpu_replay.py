"""The engine against the plain implementation, in every way of cutting the work:
each request alone and whole; the last 32 tokens one by one; batches of unequal lengths
whose shorter requests end earlier, one batch after another so that slots and pages are
used again.  In float32 and in bfloat16."""
import numpy as np
import pytest
import torch

from helpers import TINY, assert_close, model_folder, plain_logits, random_tokens

pytestmark = pytest.mark.gpu

CASES = [("a", "float32"), ("b", "float32"), ("a", "bfloat16"), ("b", "bfloat16"),
         ("c", "float32"), ("c", "bfloat16"), ("d", "bfloat16"), ("d", "float32")]
LENGTHS = {"a": [60, 7, 33, 64, 1, 41], "b": [100, 5, 11, 2, 77, 128, 64],
           "c": [130, 40, 257, 64, 3], "d": [200, 65, 31, 129]}


def storage_of(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@pytest.fixture(scope="module")
def engines():
    from gguf2bin_b200.engine import Engine, Model
    made = {}

    def get(name, dtype, max_tokens=2048):
        key = (name, dtype, max_tokens)
        if key not in made:
            model = Model.from_folder(model_folder(name, storage_of(dtype)), dtype=dtype)
            made[key] = Engine(model, max_tokens=max_tokens)
        return made[key]
    return get


def requests_of(name):
    return [random_tokens(name, n, i) for i, n in enumerate(LENGTHS[name])]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole(engines, name, dtype):
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    for i, toks in enumerate(requests_of(name)):
        seq = eng.open_sequence()
        logits = eng.step([StepEntry(seq, toks, range(len(toks)))]).cpu().numpy()
        eng.close_sequence(seq)
        assert_close(logits, plain_logits(name, storage_of(dtype), toks), dtype,
                     f"{name}/{dtype} request {i} whole")


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_one_by_one(engines, name, dtype):
    from gguf2bin_b200.engine import StepEntry
    eng = engines(name, dtype)
    for i, toks in enumerate(requests_of(name)):
        if len(toks) <= 32:
            continue
        ref = plain_logits(name, storage_of(dtype), toks)
        seq = eng.open_sequence()
        head = len(toks) - 32
        got = [eng.step([StepEntry(seq, toks[:head], range(head))]).cpu().numpy()]
        for t in range(head, len(toks)):
            got.append(eng.step([StepEntry(seq, [toks[t]], [0])]).cpu().numpy())
        eng.close_sequence(seq)
        assert_close(np.concatenate(got), ref, dtype, f"{name}/{dtype} request {i} last-32")


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_with_reuse(engines, name, dtype):
    """Batches of three requests: their prompts (all but the last 8 tokens, at least one)
    in one step, then one token each; shorter requests end earlier.  The cache is just
    large enough for one batch, so every batch reuses the slots and pages of the last."""
    from gguf2bin_b200.engine import StepEntry
    reqs = requests_of(name)
    batches = [reqs[i:i + 3] for i in range(0, len(reqs), 3)]
    need = max(sum(-(-len(t) // 64) * 64 for t in b) for b in batches)
    eng = engines(name, dtype, need)
    for bi, batch in enumerate(batches):
        seqs = [eng.open_sequence() for _ in batch]
        heads = [max(1, len(t) - 8) for t in batch]
        got = [[] for _ in batch]
        out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(seqs, batch, heads)])
        out = out.cpu().numpy()
        o = 0
        for j, h in enumerate(heads):
            got[j].append(out[o:o + h])
            o += h
        done = list(heads)
        live = [j for j in range(len(batch)) if done[j] < len(batch[j])]
        for j in range(len(batch)):
            if j not in live:
                eng.close_sequence(seqs[j])
        while live:
            out = eng.step([StepEntry(seqs[j], [batch[j][done[j]]], [0]) for j in live])
            out = out.cpu().numpy()
            for r, j in enumerate(live):
                got[j].append(out[r:r + 1])
                done[j] += 1
            for j in [j for j in live if done[j] == len(batch[j])]:
                eng.close_sequence(seqs[j])
            live = [j for j in live if done[j] < len(batch[j])]
        for j, toks in enumerate(batch):
            assert_close(np.concatenate(got[j]), plain_logits(name, storage_of(dtype), toks),
                         dtype, f"{name}/{dtype} batch {bi} request {j}")
    assert eng.cache.table.pages.n_held == 0 and eng.cache.table.slots.n_held == 0
