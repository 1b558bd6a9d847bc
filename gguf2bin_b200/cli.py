"""Command line in the manner of the reference's (src/main.c:65-94, 498-507 of
AnonymoDGH/gguf2bin): sub-commands ``run``, ``bench``, ``info`` and ``synth`` with the
same option names and meanings where it has them.

    run   <model_dir> --tokens a,b,c [--tokens d,e ...] [--tokens-file FILE] [-n N] [-t TEMP]
          [--top-k K] [--top-p P] [--repeat-penalty R] [-c N | --ctx N] [--seed S]
          [--dtype D] [--stop id,id] [--ignore-eos]
    bench <model_dir> [-n N] [-c N] [--dtype D]
    info  <model_dir>
    synth <out_dir> --config config.json [--seed S] [--dtype D]

What differs, and why: a model is a folder (config.json + safetensors), not a G2BX or
GGUF file; there is no tokenizer, so prompts are token ids (``--tokens``, which may be
given several times for a batch, and ``--tokens-file``, one request per line, for prompts
too long to type: the reference caps a command-line prompt at 1,024 ids, src/main.c:291-294)
and text prompts are refused; sampling is seeded
(``--seed``) instead of taking the clock; ``synth`` writes random weights, not zeros.
The reference's CPU memory options (--q8-kv, --f32-kv, --max-ram, --swap, --fast,
--threads) and --bos have no meaning here and are refused with that explanation.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

_CPU_ONLY = {"--q8-kv", "--f32-kv", "--max-ram", "--swap", "--fast", "--threads", "--bos"}


def _ids(text: str) -> list:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be integers separated by commas: {text!r}")


class CommandLineError(ValueError):
    """An argument that cannot be used; the message is printed as one line."""


def read_tokens_file(path) -> list:
    """One request per line: ids separated by commas or blanks; empty lines and lines that
    start with ``#`` are skipped."""
    try:
        lines = Path(path).read_text().splitlines()
    except OSError as e:
        raise CommandLineError(f"--tokens-file {path}: {e.strerror or e}") from None
    prompts = []
    for no, line in enumerate(lines, 1):
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        try:
            prompts.append([int(t) for t in line.replace(",", " ").split()])
        except ValueError:
            raise CommandLineError(f"--tokens-file {path}, line {no}: token ids must be integers") from None
    if not prompts:
        raise CommandLineError(f"--tokens-file {path}: no request in the file")
    return prompts


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gguf2bin_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    run = sub.add_parser("run", help="generate from token ids")
    run.add_argument("model")
    run.add_argument("text", nargs="*", help=argparse.SUPPRESS)
    run.add_argument("-n", type=int, default=64, help="tokens to generate (default 64)")
    run.add_argument("-t", type=float, default=0.7, help="temperature (0 = greedy, default 0.7)")
    run.add_argument("--top-k", type=int, default=40, help="top-k (default 40)")
    run.add_argument("--top-p", type=float, default=0.9, help="nucleus p (default 0.9)")
    run.add_argument("--repeat-penalty", type=float, default=1.1, help="(default 1.1)")
    run.add_argument("--tokens", type=_ids, action="append", default=[],
                     help="prompt ids a,b,c; repeat the option for a batch")
    run.add_argument("--tokens-file", action="append", default=[], metavar="FILE",
                     help="a file with one request per line (ids separated by commas or blanks)")
    run.add_argument("-c", "--ctx", type=int, default=0, help="context limit (default: the model's)")
    run.add_argument("--seed", type=int, default=0)
    run.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    run.add_argument("--stop", type=_ids, default=None, help="stop ids (default: the model's eos)")
    run.add_argument("--ignore-eos", action="store_true")

    bench = sub.add_parser("bench", help="time single-token steps")
    bench.add_argument("model")
    bench.add_argument("-n", type=int, default=32, help="steps (default 32)")
    bench.add_argument("-c", "--ctx", type=int, default=0)
    bench.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])

    info = sub.add_parser("info", help="print the model's configuration and tensors")
    info.add_argument("model")

    synth = sub.add_parser("synth", help="write a model folder with random weights")
    synth.add_argument("out")
    synth.add_argument("--config", required=True, help="a config.json to take the sizes from")
    synth.add_argument("--seed", type=int, default=0)
    synth.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    return ap


def cmd_run(a) -> int:
    if a.text:
        print("run: text prompts need a tokenizer, which this library does not have; "
              "pass token ids with --tokens a,b,c", file=sys.stderr)
        return 1
    from .api import LLM
    prompts = list(a.tokens)
    for path in a.tokens_file:
        prompts += read_tokens_file(path)
    prompts = prompts or [[1]]                       # src/main.c:312: default prompt [1]
    llm = LLM(a.model, dtype=a.dtype,
              max_tokens=sum(-(-(len(p) + a.n) // 64) * 64 for p in prompts))
    print(llm.model.describe(), file=sys.stderr)
    outs = llm.generate(prompts, n=a.n, temperature=a.t, top_k=a.top_k, top_p=a.top_p,
                        repeat_penalty=a.repeat_penalty, seed=a.seed, stop_ids=a.stop,
                        ignore_eos=a.ignore_eos, ctx=a.ctx or None)
    for p, o in zip(prompts, outs):
        print(" ".join(str(t) for t in list(p) + o.tokens))
        if o.finish_reason == "context":
            print("run: context full; stop", file=sys.stderr)
    return 0


def cmd_bench(a) -> int:
    """As the reference's bench (src/main.c:469-496): one warm-up step, then ``n`` timed
    single-token steps of one sequence, token i % vocab at position i."""
    import torch
    from .engine import Engine, Model, StepEntry
    model = Model.from_folder(a.model, dtype=a.dtype)
    ctx = min(a.ctx or model.spec.max_positions, model.spec.max_positions)
    n = min(a.n, ctx - 1)
    eng = Engine(model, max_tokens=n + 1)
    seq = eng.open_sequence()
    eng.step([StepEntry(seq, (1,), (0,))])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n):
        eng.step([StepEntry(seq, (i % model.vocab,), (0,))])
    torch.cuda.synchronize()
    sec = max(time.perf_counter() - t0, 1e-9)
    print(f"bench: {n} tokens in {sec:.4f}s -> {n / sec:.1f} tok/s  (dim={model.hidden} "
          f"L={len(model.spec.layers)} ctx={ctx})", file=sys.stderr)
    return 0


def cmd_info(a) -> int:
    from .config import model_spec_from_folder, read_config_json
    from .engine.model import expected_tensors
    from .weights import open_model_files
    cfg = read_config_json(a.model)
    spec = model_spec_from_folder(a.model)
    print(f"architecture {spec.architecture}: {len(spec.layers)} layers, width {spec.hidden_size}, "
          f"vocab {spec.vocab_size}, max positions {spec.max_positions}")
    for k in sorted(cfg):
        print(f"  {k} = {cfg[k]!r}")
    files = open_model_files(a.model)
    found = {n: e for f in files for n, e in f.entries.items()}
    exp = expected_tensors(spec)
    print(f"tensors: {len(found)} in the folder, {len(exp)} named by the model")
    for n, e in found.items():
        mark = "" if n in exp else "   (not used)"
        print(f"  {n}  {e.dtype}{list(e.shape)}{mark}")
    return 0


def cmd_synth(a) -> int:
    from .weights import write_random_model
    cfg = json.loads(Path(a.config).read_text())
    out = write_random_model(a.out, cfg, a.seed, a.dtype)
    print(f"synth: wrote {out}/config.json and model.safetensors (seed {a.seed}, {a.dtype})",
          file=sys.stderr)
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    for arg in argv:
        if arg in _CPU_ONLY:
            print(f"{arg}: an option of the reference's CPU runtime (memory budget, threads or "
                  "tokenizer) that has no meaning for this GPU library; use --dtype for precision "
                  "and -c for the context", file=sys.stderr)
            return 1
    a = _parser().parse_args(argv)
    command = {"run": cmd_run, "bench": cmd_bench, "info": cmd_info, "synth": cmd_synth}[a.command]
    try:
        return command(a)
    except _expected_errors() as e:
        # what a user can cause (a bad folder, a prompt that does not fit, no GPU): one line, no traceback
        first, *rest = str(e).splitlines() or [type(e).__name__]
        print(f"{a.command}: {first}", file=sys.stderr)
        for line in rest:
            print(line, file=sys.stderr)
        return 1


def _expected_errors() -> tuple:
    from .cache.pool import CacheError
    from .config import ConfigError
    from .csrc.build import KernelBuildError, KernelError
    from .engine.generate import GenerationError
    from .engine.step import StepError
    from .weights import WeightsError
    return (CommandLineError, CacheError, ConfigError, KernelBuildError, KernelError, GenerationError,
            StepError, WeightsError, FileNotFoundError)


if __name__ == "__main__":
    sys.exit(main())
