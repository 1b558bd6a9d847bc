#!/usr/bin/env python3
"""Decode and prefill throughput of gguf2bin_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|ragged8|b64] [--batch B] [--layers L] [--context C]
                    [--no-points] [--sizes 0.6b|8b|14b]

The default run has the layer sizes of Qwen3-0.6B (28 layers, width 1024, 16/8 heads of
128, feed-forward 3072, vocabulary 151936, tied embeddings) with random bfloat16
weights, a batch of 8 and a context of 4096: every sequence is prefilled with random
token ids up to position 2048 and then decoded.  A "step" is one decode step of the
whole batch.  It prints ONE JSON line:

  value      decoded tokens per second over exactly K steps, timed on the device with CUDA
             events (the steps run back to back from a CUDA graph; sampled tokens stay on
             the device)
  e2e        the same through the Python entry point (LLM.generate; `default_sampling`: with its own
             sampling parameters instead of greedy): token ids go in
             from pinned host memory and come back to the host every step; the median of
             three calls (each with its own prompts' prefill before and the set-up of its
             decode session inside the timed steps), all three listed under "runs"
  prefill    one step over a 2,048-token prompt: tokens per second, milliseconds (the median of
             three runs that replay the shape's graph; ``plain_ms`` is a run of the warm engine
             without the graph, what a shape costs when it is first seen; ``first_ms`` the very
             first run, which also builds scratch buffers and loads kernels), and the fraction of
             the tensor-core peak its flops reach
  roofline   bytes a decode step must read (every weight once, the cache of the live
             requests) divided by its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (fewer steps), each with its step time
             and its own roofline figures

``--workload ragged8`` runs the workload of the Qwen3-8B configuration (all 36 layers): eight
prompts with lengths drawn uniformly from [128, 2048] (seeded) in ONE ragged prompt step, whose
tokens per second go under ``prefill``, then 256 decode steps.  ``--workload b64`` runs that of
the Qwen3-14B configuration (all 40 layers): 64 prompts of 512 tokens in one prompt step, then
decoding to a context of 2,048.  The weights are made in device memory (no folder is written).

Peaks come from MEASURED_PEAKS.json beside this file when present, else from the
fallback figures 6.65 TB/s and 1.59 PFLOP/s.  Inputs are synthetic.  Between timed steps
nothing is flushed: a step reads more than a gigabyte of weights and cache, far more than
the 126 MB of L2.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_0P6B = dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=3072,
                  num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                  head_dim=128, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
                  tie_word_embeddings=True, max_position_embeddings=40960)
# the layer sizes of Qwen3-8B and Qwen3-14B, for `--sizes` (not the default run)
OTHER_SIZES = {
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
               num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, tie_word_embeddings=False),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        source="measured")
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None,
                    sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons),
                    samples=len(sm))


def model_bytes_and_flops(cfg: dict, n_layers: int):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    nq, nk = nh * hd, nkv * hd
    layer = H * (nq + 2 * nk) + nq * H + 2 * H * I + I * H            # matrix parameters of a layer
    vectors = 2 * H + 2 * hd
    weight_bytes = 2 * (n_layers * (layer + vectors) + H + V * H)       # bf16; lm_head read once
    kv_bytes_per_token = 2 * nk * 2 * n_layers                          # K and V, bf16, all layers
    return dict(layer_params=layer, weight_bytes=weight_bytes, kv_bytes_per_token=kv_bytes_per_token,
                nq=nq)


def prefill_flops(cfg: dict, n_layers: int, lengths) -> float:
    """Flops of one prompt step over sequences of these lengths, logits at each one's last place."""
    m = model_bytes_and_flops(cfg, n_layers)
    total = float(sum(lengths))
    linear = 2.0 * total * n_layers * m["layer_params"]
    attention = sum(n_layers * 4.0 * m["nq"] * T * (T + 1) / 2 for T in lengths)
    head = 2.0 * cfg["vocab_size"] * cfg["hidden_size"] * len(lengths)
    return linear + attention + head


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def timed_prompt_step(llm, prompts, repeats: int):
    """Milliseconds of ONE step over all the prompts (logits at each last place), device-timed:
    (the very first run, which also builds scratch buffers and loads kernels; the median of the
    last ``repeats`` runs, which replay the shape's graph; a run of the warm engine without the
    graph, which is what a shape costs the first time it is seen)."""
    import gc
    import torch
    from gguf2bin_b200.engine import StepEntry
    times = []
    # the plain run's time is the host's; a collection of Python's cycle collector in the middle of it
    # (this program holds hundreds of thousands of token ids in lists) adds a millisecond or two
    gc.collect()
    gc.disable()
    for i in range(3 + repeats + 1):
        if i == 3 + repeats:                       # once more without the graph: a warm engine's plain run,
            graphs, llm.engine.step_graphs = llm.engine.step_graphs, False     # what a shape seen for the first time costs
        seqs = [llm.open_sequence() for _ in prompts]
        for s, p in zip(seqs, prompts):
            llm.engine.cache.reserve(s, len(p))
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        llm.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(seqs, prompts)])
        e1.record()
        torch.cuda.synchronize()
        for s in seqs:
            llm.close_sequence(s)
        times.append(e0.elapsed_time(e1))
    llm.engine.step_graphs = graphs
    gc.enable()
    return times[0], statistics.median(times[3:-1]), times[-1]


def decode_device_timed(llm, prompts, steps: int, warmup: int, vocab: int, whole_batch_prefill: bool):
    """Decodes ``steps`` steps after the prompts and ``warmup`` untimed steps: (seconds for
    exactly ``steps`` steps, launches per step, mean context over the timed steps), timed on
    the device.  The prompts are prefilled one sequence per step, or all in one ragged step."""
    import torch
    from gguf2bin_b200.engine import DecodeSession, StepEntry
    from gguf2bin_b200.sampling import Sampler, SamplingParams
    eng = llm.engine
    batch = len(prompts)
    seqs = [eng.open_sequence() for _ in range(batch)]
    try:
        for s, p in zip(seqs, prompts):
            eng.cache.reserve(s, len(p) + warmup + steps + 1)
        if whole_batch_prefill:
            eng.step([StepEntry(s, p, ()) for s, p in zip(seqs, prompts)])
        else:
            for s, p in zip(seqs, prompts):
                eng.step([StepEntry(s, p, ())])
        sampler = Sampler(eng.cache.seq_state, eng.device)
        session = DecodeSession(eng, seqs, sampler, SamplingParams.plain(0.0), use_graph=True,
                                eager_steps=1)
        session.set_tokens(random_prompts(1, batch, vocab, 7)[0])
        for _ in range(warmup):
            session.run()
        torch.cuda.synchronize()
        start = sum(s.length for s in seqs) / batch
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            session.run()
        t1.record()
        torch.cuda.synchronize()
        eng.check()
        return t0.elapsed_time(t1) / 1e3, session.launches_per_step, start + steps / 2.0
    finally:
        for s in seqs:
            eng.close_sequence(s)


def hbm_roofline(sizes: dict, batch: int, mean_ctx: float, sec_per_step: float, pk: dict) -> dict:
    """Bytes a decode step has to read (every weight once, the cache of the live requests)
    over its time, against the copy bandwidth."""
    step_bytes = sizes["weight_bytes"] + batch * mean_ctx * sizes["kv_bytes_per_token"]
    achieved = step_bytes / sec_per_step / 1e9
    return dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s",
                frac=achieved / pk["hbm_gbs"], peaks=pk["source"])


WORKLOADS = {
    # name: (sizes, batch, what it is)
    "decode": ("0.6b", 8, "every sequence prefilled to half the context, then decoded"),
    "ragged8": ("8b", 8, "8 prompts with lengths uniform in [128, 2048] in ONE prompt step, then 256 decode steps"),
    "b64": ("14b", 64, "64 prompts of 512 tokens in one prompt step, decoded to a context of 2048"),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="decode steps timed (default: 512; the workload's own for ragged8 and b64)")
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=sorted(WORKLOADS),
                    help="decode: the default run; ragged8 / b64: the two larger configurations' own workloads")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--sizes", default=None, choices=["0.6b"] + sorted(OTHER_SIZES),
                    help="layer sizes: Qwen3-0.6B, or those of Qwen3-8B / 14B (default: the workload's)")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the prompt of the prefill figure (decode workload; default 2048)")
    a = ap.parse_args()

    if a.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AnonymoDGH/gguf2bin is a C99 Makefile project without setup.py or "
                          "pyproject.toml, so pip cannot install it into baseline/_ref; it has no "
                          "GPU code and no batching"}))
        return 0
    if a.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {a.gpus} is not supported")
        return 2
    if a.warmup < 3:
        a.warmup = 3

    import numpy as np
    import torch
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.api import LLM

    w_sizes, w_batch, w_what = WORKLOADS[a.workload]
    a.sizes = a.sizes or w_sizes
    a.batch = a.batch or w_batch
    cfg = dict(QWEN3_0P6B)
    cfg.update(OTHER_SIZES.get(a.sizes, {}))
    full_layers = cfg["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg["num_hidden_layers"] = a.layers
    name = {"0.6b": "Qwen3-0.6B", "8b": "Qwen3-8B", "14b": "Qwen3-14B"}[a.sizes]
    pk = peaks()
    sizes = model_bytes_and_flops(cfg, a.layers)
    vocab = cfg["vocab_size"]

    # ---- the workload's prompts and steps ----------------------------------------------------
    if a.workload == "decode":
        start_ctx = a.context // 2
        steps = min(a.steps or 512, a.context - start_ctx - 1)
        decode_prompts = random_prompts(a.batch, start_ctx - a.warmup, vocab, 100)
        prefill_prompts = random_prompts(1, a.prefill_tokens, vocab, 1)
        seq_len = a.context
        points_wanted = not a.no_points
        max_batch = max(64 if points_wanted else a.batch, a.batch)
        max_tokens = max(max_batch * (a.context + 64), a.prefill_tokens + 64)
    elif a.workload == "ragged8":
        lengths = np.random.default_rng(2024).integers(128, 2049, a.batch).tolist()
        steps = a.steps or 256
        decode_prompts = [random_prompts(1, n, vocab, 300 + i)[0] for i, n in enumerate(lengths)]
        prefill_prompts = decode_prompts
        seq_len = max(lengths) + a.warmup + steps
        points_wanted, max_batch = False, a.batch
        max_tokens = sum(-(-(n + a.warmup + steps + 2) // 64) * 64 for n in lengths) + 64
    else:
        a.context = 2048
        steps = min(a.steps or 10 ** 9, a.context - 512 - a.warmup)
        decode_prompts = random_prompts(a.batch, 512, vocab, 500)
        prefill_prompts = decode_prompts
        seq_len = a.context
        points_wanted, max_batch = False, a.batch
        max_tokens = a.batch * (a.context + 64)

    free0, total_mem = torch.cuda.mem_get_info()
    llm = LLM.random(cfg, seed=0, dtype="bfloat16", max_tokens=max_tokens, max_seqs=max_batch + 1)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()

    # ---- prefill: one step over the prompts, logits at each last place ------------------------
    pre_first, pre, pre_plain = timed_prompt_step(llm, prefill_prompts, repeats=3)
    pre_lengths = [len(p) for p in prefill_prompts]
    pre_tokens = sum(pre_lengths)
    pre_flops = prefill_flops(cfg, a.layers, pre_lengths)
    prefill = dict(value=pre_tokens / (pre / 1e3), tokens=pre_tokens, ms=pre,
                   frac=pre_flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12),
                   first_ms=pre_first, plain_ms=pre_plain, sequences=len(pre_lengths))

    # ---- decode, device-timed -----------------------------------------------------------------
    clocks = ClockSampler()
    clocks.start()
    sec, per_step, mean_ctx = decode_device_timed(llm, decode_prompts, steps, a.warmup, vocab,
                                                  whole_batch_prefill=a.workload != "decode")
    clock_info = clocks.stop()
    value = a.batch * steps / sec
    roofline = hbm_roofline(sizes, a.batch, mean_ctx, sec / steps, pk)

    # ---- decode through the Python entry point, host tokens in and out -------------------------
    e2e_steps = min(steps, 256)
    e2e_prompts = [p + [1] * a.warmup for p in decode_prompts]     # the same lengths as the timed steps start from
    llm.generate(e2e_prompts[:1], n=4, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                 ignore_eos=True)
    e2e_runs = []                      # three whole calls; the median is reported, all are listed
    for _ in range(3):
        llm.generate(e2e_prompts, n=e2e_steps + 1, temperature=0.0, top_k=0, top_p=1.0,
                     repeat_penalty=1.0, ignore_eos=True, max_batch=a.batch)
        acct = llm.last_decode
        e2e_runs.append((acct["tokens"] / acct["seconds"], acct["steps"]))
    e2e_value, e2e_count = sorted(e2e_runs)[1]
    # the same call with the entry point's own sampling parameters (temperature 0.7, top-k 40,
    # top-p 0.9, repeat penalty 1.1: what a user who sets nothing gets); the second of two calls
    sampled = []
    for _ in range(2):
        llm.generate(e2e_prompts, n=e2e_steps + 1, ignore_eos=True, max_batch=a.batch)
        sampled.append(llm.last_decode["tokens"] / llm.last_decode["seconds"])
    e2e = dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=4 * a.batch,
               d2h_bytes_per_step=4 * a.batch, steps=e2e_count,
               runs=[round(v, 1) for v, _ in e2e_runs], default_sampling=round(sampled[-1], 1),
               graphs_captured=llm.engine.graph_captures)

    # ---- other batch sizes ------------------------------------------------------------------------
    points = {}
    if points_wanted:
        room = a.context - start_ctx - 1
        for b, k in ((1, min(room, 256)), (64, min(room, 128))):    # their own step counts, whatever --steps says:
            warm = max(a.warmup, 16)                                # twenty steps of 0.7 ms mostly measure the clocks settling
            s, _, ctx_b = decode_device_timed(llm, random_prompts(b, start_ctx - warm, vocab, 100), k,
                                              warm, vocab, whole_batch_prefill=False)
            r = hbm_roofline(sizes, b, ctx_b, s / k, pk)
            points[f"decode_b{b}"] = b * k / s
            points[f"decode_b{b}_ms_per_step"] = s / k * 1e3
            points[f"decode_b{b}_gbs"] = r["achieved"]
            points[f"decode_b{b}_frac"] = r["frac"]

    first_ctx = mean_ctx - steps / 2.0
    out = {
        "metric": f"decode tokens/s ({name} sizes, random weights, batch {a.batch}, "
                  f"context {first_ctx:.0f}->{first_ctx + steps:.0f})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": a.warmup,
        "ms_per_step": sec / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{name} sizes, random weights", "workload": f"{a.workload}: {w_what}",
                   "global_batch": a.batch,
                   "seq_len": seq_len, "decode_from": round(first_ctx, 1), "layers": a.layers,
                   "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": vocab, "tied": bool(cfg["tie_word_embeddings"]), "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (weights + cache read every step)",
                   "sampling": "greedy on device",
                   "weights": "made on the device (Philox normal), never on disk",
                   "device_gb_free_before_after": f"{free0 / 1e9:.1f} -> {free1 / 1e9:.1f} of {total_mem / 1e9:.1f}"},
        "e2e": e2e, "gpu_launches": per_step * steps, "launches_per_step": per_step,
        "prefill": prefill, "roofline": roofline, "points": points, "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
