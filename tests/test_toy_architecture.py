"""Another architecture added from outside the package (tests/toy_hybrid.py: its own
config.json keys and tensor names, layers that alternate attention with a fixed-size-state
mixer, a scaled embedding): through the registry, the weights loader, the Python entry point,
the command line and trace replay, with no change to the package's files."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import toy_hybrid
from helpers import assert_close
from plain import qwen3_plain as P

ROOT = Path(__file__).resolve().parent.parent
ENV = dict(os.environ, GGUF2BIN_B200_PLUGINS="toy_hybrid",
           PYTHONPATH=os.pathsep.join([str(ROOT / "tests"), os.environ.get("PYTHONPATH", "")]))


def make_folder(tmp_path, storage="float32"):
    from gguf2bin_b200.weights import write_random_model
    return write_random_model(tmp_path / "toy_model", toy_hybrid.CONFIG, seed=21, dtype=storage, std=0.05)


def test_the_registry_builds_its_spec_and_tensor_list(tmp_path):
    from gguf2bin_b200.cache import KVNeed, StateNeed
    from gguf2bin_b200.config import ConfigError, model_spec_from_dict, model_spec_from_folder
    from gguf2bin_b200.engine.model import expected_tensors
    folder = make_folder(tmp_path)
    spec = model_spec_from_folder(folder)
    assert spec.architecture == toy_hybrid.ARCHITECTURE and [l.mixer.kind for l in spec.layers] == \
        ["gqa_attention", "toy_leaky_state", "gqa_attention"]
    names = set(expected_tensors(spec))
    assert {"wte", "ln_f", "blocks.1.mix.leak", "blocks.0.att.qn", "blocks.2.ffn.d"} <= names
    _, W = P.read_model_folder(folder)
    assert set(W) == names - {"unused_head"}
    with pytest.raises(ConfigError, match="pattern"):
        model_spec_from_dict({**toy_hybrid.CONFIG, "pattern": "AX"})
    with pytest.raises(ConfigError, match="theta"):
        model_spec_from_dict({k: v for k, v in toy_hybrid.CONFIG.items() if k != "theta"})
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "gguf2bin_b200"), "info", str(folder)], env=ENV,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "ToyHybridForCausalLM: 3 layers, width 80" in out.stdout and "(not used)" not in out.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_it_steps_and_generates(tmp_path, dtype):
    from gguf2bin_b200.api import LLM, StepEntry
    from gguf2bin_b200.cache import StateView
    storage = "float32" if dtype == "float32" else "bfloat16"
    folder = make_folder(tmp_path, storage)
    cfg, W = P.read_model_folder(folder)
    llm = LLM(folder, dtype=dtype, max_tokens=1024)
    assert isinstance(llm.engine.cache.view(1), StateView) and len(llm.engine.cache.groups) == 2
    rng = np.random.default_rng(3)
    reqs = [rng.integers(0, cfg["vocab"], n).tolist() for n in (70, 5, 33)]
    # unequal batch: prompts but for the last four tokens in one step, then one token each
    seqs = [llm.open_sequence() for _ in reqs]
    heads = [len(t) - 4 for t in reqs]
    got = [[] for _ in reqs]
    out = llm.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
    o = 0
    for j, h in enumerate(heads):
        got[j].append(out[o:o + h])
        o += h
    for d in range(4):
        out = llm.step([StepEntry(s, [t[h + d]], [0]) for s, t, h in zip(seqs, reqs, heads)]).cpu().numpy()
        for j in range(len(reqs)):
            got[j].append(out[j:j + 1])
    for s in seqs:
        llm.close_sequence(s)
    for j, toks in enumerate(reqs):
        assert_close(np.concatenate(got[j]), toy_hybrid.plain_forward(cfg, W, toks), dtype, f"request {j}")
    if dtype == "float32":          # greedy generation, sequences that end at different steps
        first = int(np.argmax(toy_hybrid.plain_forward(cfg, W, reqs[1])[-1]))
        outs = llm.generate(reqs, n=7, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_ids=[first])
        assert outs[1].finish_reason == "stop" and outs[1].tokens == []
        for toks, o in zip(reqs, outs):
            seq = list(toks)
            for t in o.tokens:
                assert t == int(np.argmax(toy_hybrid.plain_forward(cfg, W, seq)[-1]))
                seq.append(t)
        # six sequences run as steps of eight rows: the rows beyond them fold their tokens into
        # the spare slot's state, not into a sequence's
        more = reqs + [r[:k] for r, k in zip(reqs, (9, 3, 20))]
        for toks, o in zip(more, llm.generate(more, n=5, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                                              ignore_eos=True)):
            seq = list(toks)
            for t in o.tokens:
                assert t == int(np.argmax(toy_hybrid.plain_forward(cfg, W, seq)[-1]))
                seq.append(t)


@pytest.mark.gpu
def test_the_programs_know_it_through_the_plugin_variable(tmp_path):
    folder = make_folder(tmp_path)
    cfg, W = P.read_model_folder(folder)
    toks = [5, 17, 3, 99, 150, 7, 11]
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "gguf2bin_b200"), "run", str(folder), "--tokens",
                          ",".join(map(str, toks)), "-n", "5", "-t", "0", "--repeat-penalty", "1",
                          "--dtype", "float32"], env=ENV, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [int(t) for t in out.stdout.split()]
    seq = list(toks)
    for t in ids[len(toks):]:
        assert t == int(np.argmax(toy_hybrid.plain_forward(cfg, W, seq)[-1]))
        seq.append(t)
    assert len(ids) == len(toks) + 5
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:5], "want": [0, 4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[5:6], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[6:], "want": [0]}], "end": ["a"]}]
    out_dir = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(out_dir), "--max-tokens", "64"], env=ENV,
                          input="".join(json.dumps(s) + "\n" for s in steps), text=True, capture_output=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ref = toy_hybrid.plain_forward(cfg, W, toks)
    got = np.concatenate([np.fromfile(out_dir / f"{i}.f32", "<f4").reshape(-1, cfg["vocab"]) for i in range(3)])
    assert_close(got, ref[[0, 4, 5, 6]], "float32", "trace replay of the toy architecture")
    # without the variable the architecture is unknown, and the program says so in one line
    bare = {k: v for k, v in ENV.items() if k != "GGUF2BIN_B200_PLUGINS"}
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "gguf2bin_b200"), "info", str(folder)], env=bare,
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 1 and "not registered" in out.stderr and "Traceback" not in out.stderr
