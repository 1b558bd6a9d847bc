"""The command line (bin/gguf2bin_b200), started as a program the way the reference's
``make test`` starts its own (Makefile:35-40 of AnonymoDGH/gguf2bin: synth, info, run,
bench, one after another on the model that synth wrote)."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import TINY, random_tokens
from plain import qwen3_plain as P

ROOT = Path(__file__).resolve().parent.parent
PROGRAM = [sys.executable, str(ROOT / "bin" / "gguf2bin_b200")]


def cli(*args, ok=True):
    p = subprocess.run(PROGRAM + [str(a) for a in args], capture_output=True, text=True, timeout=600)
    if ok:
        assert p.returncode == 0, f"{args}: exit {p.returncode}\n{p.stderr[-2000:]}"
    return p


def synth(tmp_path, name, **patch):
    cfg = tmp_path / f"{name}.json"
    cfg.write_text(json.dumps({**TINY[name], **patch}))
    folder = tmp_path / f"model_{name}"
    p = cli("synth", folder, "--config", cfg, "--seed", 5, "--dtype", "float32")
    assert "synth: wrote" in p.stderr
    return folder


def plain_greedy(folder, prompt, n):
    cfg, W = P.read_model_folder(folder)
    toks = list(prompt)
    for _ in range(n):
        toks.append(P.greedy(P.forward(cfg, W, toks, np.float32)[-1]))
    return toks


# ---- without a GPU ------------------------------------------------------------------------
def test_synth_and_info(tmp_path):
    folder = synth(tmp_path, "b")
    assert (folder / "config.json").is_file() and (folder / "model.safetensors").is_file()
    out = cli("info", folder).stdout
    d = TINY["b"]
    assert f"{d['num_hidden_layers']} layers" in out and f"width {d['hidden_size']}" in out
    assert f"vocab {d['vocab_size']}" in out and "rms_norm_eps = 1e-05" in out
    assert "model.layers.2.self_attn.q_norm.weight" in out and "(not used)" not in out
    assert out.count("F32[") == len(P.read_model_folder(folder)[1])


def test_refusals_are_one_line(tmp_path):
    folder = synth(tmp_path, "a")
    for flag in ("--q8-kv", "--swap", "--threads"):
        p = cli("run", folder, flag, ok=False)
        assert p.returncode == 1 and "CPU runtime" in p.stderr and "Traceback" not in p.stderr
    p = cli("run", folder, "hello", "world", ok=False)
    assert p.returncode == 1 and "tokenizer" in p.stderr and "Traceback" not in p.stderr
    p = cli("run", folder, "--tokens", "1,x", ok=False)
    assert p.returncode == 2 and "integers" in p.stderr
    p = cli("run", folder, "--tokens-file", tmp_path / "absent.txt", ok=False)
    assert p.returncode == 1 and "absent.txt" in p.stderr and "Traceback" not in p.stderr
    bad = tmp_path / "bad.txt"
    bad.write_text("1 2 3\n4, five\n")
    p = cli("run", folder, "--tokens-file", bad, ok=False)
    assert p.returncode == 1 and "line 2" in p.stderr and "Traceback" not in p.stderr
    p = cli("info", tmp_path / "no_such_model", ok=False)
    assert p.returncode == 1 and "no such file" in p.stderr.lower() and "Traceback" not in p.stderr
    (folder / "model.safetensors").write_bytes(b"\x00" * 4)
    p = cli("info", folder, ok=False)
    assert p.returncode == 1 and "Traceback" not in p.stderr


def test_tokens_file_format(tmp_path):
    from gguf2bin_b200.cli import CommandLineError, read_tokens_file
    f = tmp_path / "t.txt"
    f.write_text("# two requests\n1, 2,3\n\n  7 8\t9  \n")
    assert read_tokens_file(f) == [[1, 2, 3], [7, 8, 9]]
    f.write_text("\n# nothing\n")
    with pytest.raises(CommandLineError, match="no request"):
        read_tokens_file(f)


def test_run_without_a_gpu_says_so_in_one_line(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this box has a GPU")
    p = cli("run", synth(tmp_path, "a"), "--tokens", "1,2,3", "-n", 2, ok=False)
    assert p.returncode == 1 and "no CUDA device" in p.stderr and "Traceback" not in p.stderr


# ---- on the GPU ---------------------------------------------------------------------------
@pytest.mark.gpu
def test_synth_info_run_bench_as_programs(tmp_path):
    folder = synth(tmp_path, "b")
    cli("info", folder)
    prompts = [random_tokens("b", n, 800 + i) for i, n in enumerate([5, 11, 2])]
    args = []
    for p in prompts:
        args += ["--tokens", ",".join(map(str, p))]
    out = cli("run", folder, *args, "-n", 9, "-t", 0, "--repeat-penalty", 1, "--dtype", "float32",
              "--ignore-eos")
    lines = [[int(t) for t in l.split()] for l in out.stdout.strip().splitlines()]
    assert lines == [plain_greedy(folder, p, 9) for p in prompts]
    assert "Qwen3ForCausalLM" in out.stderr
    # the same requests from a file, in bfloat16 with the reference's default sampling: it runs
    # and prints as many ids as asked for
    f = tmp_path / "requests.txt"
    f.write_text("\n".join(" ".join(map(str, p)) for p in prompts) + "\n")
    out = cli("run", folder, "--tokens-file", f, "-n", 6, "--seed", 3, "--ignore-eos")
    got = [[int(t) for t in l.split()] for l in out.stdout.strip().splitlines()]
    assert [g[:len(p)] for g, p in zip(got, prompts)] == prompts
    assert [len(g) - len(p) for g, p in zip(got, prompts)] == [6, 6, 6]
    b = cli("bench", folder, "-n", 8)
    assert "bench: 8 tokens in" in b.stderr and "tok/s" in b.stderr
    # a stop id from generation_config.json ends a request early
    first = lines[0][len(prompts[0])]
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [first]}))
    out = cli("run", folder, "--tokens", ",".join(map(str, prompts[0])), "-n", 9, "-t", 0,
              "--repeat-penalty", 1, "--dtype", "float32")
    assert [int(t) for t in out.stdout.split()] == prompts[0]


@pytest.mark.gpu
def test_a_prompt_of_2048_tokens_from_a_file(tmp_path):
    """The benchmark's prompt length cannot be typed as --tokens a,b,c (the reference stops at
    1,024 ids, src/main.c:291-294); from a file it runs whole, and the ids that follow are the
    plain implementation's."""
    folder = synth(tmp_path, "d", max_position_embeddings=2304)
    prompt = random_tokens("d", 2048, 900)
    f = tmp_path / "long.txt"
    f.write_text(",".join(map(str, prompt)) + "\n")
    out = cli("run", folder, "--tokens-file", f, "-n", 3, "-t", 0, "--repeat-penalty", 1,
              "--dtype", "float32", "--ignore-eos")
    got = [int(t) for t in out.stdout.split()]
    assert got[:2048] == prompt and len(got) == 2051
    cfg, W = P.read_model_folder(folder)
    toks = list(prompt)
    for t in got[2048:]:
        row = P.forward(cfg, W, toks, np.float32)[-1]
        assert row[t] >= row.max() - 2e-5 * max(1.0, np.abs(row).max())
        toks.append(t)
