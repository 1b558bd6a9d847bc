"""The generation loop's decisions, with a backend that needs no device: its "model"
answers (last token fed * 7 + position) % vocab, so every expected output can be
written down by hand."""
import pytest

from gguf2bin_b200.engine.generate import (GenerationError, decide, generate, plan_batch,
                                           reserve_tokens)

VOCAB = 101


def rule(last_token, length):
    return (last_token * 7 + length) % VOCAB


def expected(prompt, n, stop=(), ctx=10 ** 9):
    out, length, last = [], len(prompt), prompt[-1]
    if length >= ctx:
        return out, "context", None
    while True:
        tok = rule(last, length)
        if tok in stop:
            return out, "stop", tok
        out.append(tok)
        if len(out) >= n:
            return out, "length", None
        if len(prompt) + len(out) >= ctx:
            return out, "context", None
        last, length = tok, length + 1


class FakeBackend:
    def __init__(self, n_pages=64, page_size=64, max_context=4096):
        self.page_size, self.max_context, self.n_pages = page_size, max_context, n_pages
        self.held = {}                 # handle id -> pages
        self.lengths = {}
        self.next_id = 0
        self.log = []                  # ("prefill"|"decode", batch size)
        self.streams = []

    @property
    def free_pages(self):
        return self.n_pages - sum(self.held.values())

    def open(self, stream_id, reserve):
        need = -(-reserve // self.page_size)
        assert need <= self.free_pages, "the loop opened more than fits"
        h = self.next_id
        self.next_id += 1
        self.held[h] = need
        self.lengths[h] = 0
        self.streams.append(stream_id)
        return h

    def close(self, h):
        assert h in self.held, "closed twice"
        del self.held[h]

    def prefill(self, handles, prompts):
        self.log.append(("prefill", len(handles)))
        out = []
        for h, p in zip(handles, prompts):
            assert self.lengths[h] == 0
            self.lengths[h] = len(p)
            assert self.lengths[h] <= self.held[h] * self.page_size
            out.append(rule(p[-1], len(p)))
        return out

    def decode(self, handles, tokens):
        self.log.append(("decode", len(handles)))
        out = []
        for h, t in zip(handles, tokens):
            assert h in self.held, "a finished sequence was stepped"
            self.lengths[h] += 1
            assert self.lengths[h] <= self.held[h] * self.page_size, "fed past the reservation"
            assert self.lengths[h] <= self.max_context
            out.append(rule(t, self.lengths[h]))
        return out


def test_unequal_prompts_and_early_finishers():
    be = FakeBackend()
    prompts = [[3, 4, 5], [9], [1, 2, 3, 4, 5, 6, 7], [50, 60]]
    stop = {rule(rule(9, 1), 2)}                      # request 1 stops at its second token
    outs = generate(be, prompts, 6, stop_ids=stop)
    for p, o in zip(prompts, outs):
        toks, reason, st = expected(p, 6, stop)
        assert (o.tokens, o.finish_reason, o.stop_token) == (toks, reason, st)
    assert outs[1].finish_reason == "stop" and len(outs[1].tokens) == 1
    assert be.log[0] == ("prefill", 4)
    sizes = [n for kind, n in be.log[1:]]
    assert sizes == sorted(sizes, reverse=True) and sizes[0] == 4 and sizes[-1] == 3
    assert len(be.log) == 1 + 5                       # the 6th token is never fed
    assert not be.held


def test_batches_one_after_another_reuse_the_cache():
    be = FakeBackend(n_pages=4)
    prompts = [[i + 1] * 70 for i in range(5)]        # 70 + 9 fed positions: 2 pages each
    outs = generate(be, prompts, 10)
    assert [k for k, _ in be.log if k == "prefill"] == ["prefill"] * 3
    assert [n for k, n in be.log if k == "prefill"] == [2, 2, 1]
    for p, o in zip(prompts, outs):
        assert o.tokens == expected(p, 10)[0] and o.finish_reason == "length"
    assert be.streams == [0, 1, 2, 3, 4]              # stream ids follow the requests, not the slots
    assert not be.held


def test_max_batch_and_context_limit():
    be = FakeBackend(max_context=12)
    prompts = [[5] * 10, [6] * 12, [7] * 3]
    outs = generate(be, prompts, 8, max_batch=2)
    assert [n for k, n in be.log if k == "prefill"] == [2, 1]
    for p, o in zip(prompts, outs):
        toks, reason, _ = expected(p, 8, ctx=12)
        assert (o.tokens, o.finish_reason) == (toks, reason)
    assert outs[0].finish_reason == "context" and len(outs[0].tokens) == 2
    assert outs[1].finish_reason == "context" and outs[1].tokens == []
    assert outs[2].finish_reason == "length"


def test_refusals():
    be = FakeBackend(n_pages=1, max_context=100)
    with pytest.raises(GenerationError, match="empty"):
        generate(be, [[1], []], 4)
    with pytest.raises(GenerationError, match="101 tokens"):
        generate(be, [[1] * 101], 4)
    with pytest.raises(GenerationError, match="pages"):
        generate(be, [[1] * 80], 4)
    assert not be.held
    outs = generate(be, [[1, 2]], 0)
    assert outs[0].tokens == [] and outs[0].finish_reason == "length" and not be.log


def test_decide_and_plan():
    assert decide(5, 1, 3, {5}, 10, 100) == (False, "stop")
    assert decide(4, 10, 3, {5}, 10, 100) == (True, "length")
    assert decide(4, 2, 98, {5}, 10, 100) == (True, "context")
    assert decide(4, 2, 3, {5}, 10, 100) == (True, None)
    assert reserve_tokens(10, 5, 100) == 14 and reserve_tokens(98, 50, 100) == 100
    assert plan_batch([64, 64, 64], 1, 4096, 64, 2, 8) == 2
    assert plan_batch([64, 64, 64], 2, 4096, 64, 4, 8) == 2      # 65 positions: two pages each
    assert plan_batch([10] * 9, 1, 4096, 64, 100, 4) == 4
    with pytest.raises(GenerationError):
        plan_batch([1000], 1, 4096, 64, 2, 8)
