"""How many rows a step runs (host-side decisions, no GPU): decode batches in eights, prompt steps
filled up to a multiple of 64 rows."""
from types import SimpleNamespace

from gguf2bin_b200.engine.decode import padded_rows
from gguf2bin_b200.engine.step import Engine, StepEntry


def test_decode_batches_run_their_rows_in_eights():
    assert [padded_rows(n) for n in range(1, 10)] == [1, 2, 3, 4, 8, 8, 8, 8, 16]
    assert [padded_rows(n) for n in (16, 17, 63, 64, 65, 200)] == [16, 24, 64, 64, 72, 200]
    assert all(padded_rows(n) >= n and padded_rows(n) - n < 8 for n in range(1, 300))


def _engine(graphs=True):
    padding = SimpleNamespace(slot=99, pages=[7], length=0)
    return SimpleNamespace(step_graphs=graphs, GRAPH_MIN_TOKENS=Engine.GRAPH_MIN_TOKENS,
                           PROMPT_ROW_STEP=Engine.PROMPT_ROW_STEP, _padding=padding)


def _entries(*lengths):
    return [StepEntry(SimpleNamespace(slot=i, pages=[], length=0), [1] * n, (n - 1,)) for i, n in enumerate(lengths)]


def test_prompt_steps_are_filled_up_to_a_multiple_of_64_rows():
    eng = _engine()
    for lengths in ((5,), (63,), (65,), (100, 60), (1, 1, 70), (2000, 47)):
        entries = _entries(*lengths)
        run = Engine._filled_up(eng, entries)
        assert run[:len(entries)] == entries, "the sequences' own entries stay in front, untouched"
        rows = sum(len(e.tokens) for e in run)
        assert rows % 64 == 0 and rows - sum(lengths) < 64
        assert len(run) == len(entries) + 1 and run[-1].seq is eng._padding and tuple(run[-1].want) == ()
    # nothing to add: a multiple of 64 already, one token per sequence, a model whose steps are not replayed
    for lengths in ((64,), (2048,), (100, 28), (1,), (1, 1, 1)):
        entries = _entries(*lengths)
        assert Engine._filled_up(eng, entries) is entries
    entries = _entries(50)
    assert Engine._filled_up(_engine(graphs=False), entries) is entries
