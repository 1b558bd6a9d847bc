#!/usr/bin/env python3
"""Decode and prefill throughput of gguf2bin_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--layers L] [--context C] [--no-points] [--sizes 0.6b|8b|14b]

The default run has the layer sizes of Qwen3-0.6B (28 layers, width 1024, 16/8 heads of
128, feed-forward 3072, vocabulary 151936, tied embeddings) with random bfloat16
weights, a batch of 8 and a context of 4096: every sequence is prefilled with random
token ids up to position 2048 and then decoded.  A "step" is one decode step of the
whole batch.  It prints ONE JSON line:

  value      decoded tokens per second over exactly K steps, timed on the device with CUDA
             events (the steps run back to back from a CUDA graph; sampled tokens stay on
             the device)
  e2e        the same through the Python entry point (LLM.generate): token ids go in
             from pinned host memory and come back to the host every step; the median of
             three calls (each with its own prompts' prefill before and the set-up of its
             decode session inside the timed steps), all three listed under "runs"
  prefill    one step over a 2,048-token prompt: tokens per second, milliseconds, and the
             fraction of the tensor-core peak its flops reach
  roofline   bytes a decode step must read (every weight once, the cache of the live
             requests) divided by its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (fewer steps)

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


def prefill_flops(cfg: dict, n_layers: int, T: int) -> float:
    m = model_bytes_and_flops(cfg, n_layers)
    linear = 2.0 * T * n_layers * m["layer_params"]
    attention = n_layers * 4.0 * m["nq"] * T * (T + 1) / 2
    head = 2.0 * cfg["vocab_size"] * cfg["hidden_size"]
    return linear + attention + head


def random_prompts(n: int, length: int, vocab: int, seed: int):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def decode_device_timed(llm, batch: int, start_ctx: int, steps: int, warmup: int, vocab: int):
    """(seconds for exactly `steps` steps, launches per step, mean context) on the device."""
    import torch
    from gguf2bin_b200.engine import DecodeSession, StepEntry
    from gguf2bin_b200.sampling import Sampler, SamplingParams
    eng = llm.engine
    seqs = [eng.open_sequence() for _ in range(batch)]
    try:
        plen = start_ctx - warmup
        for i, s in enumerate(seqs):
            eng.cache.reserve(s, start_ctx + steps + 1)
            eng.step([StepEntry(s, random_prompts(1, plen, vocab, 100 + i)[0], ())])
        sampler = Sampler(eng.cache.seq_state, eng.device)
        session = DecodeSession(eng, seqs, sampler, SamplingParams.plain(0.0), use_graph=True,
                                eager_steps=1)
        session.set_tokens(random_prompts(1, batch, vocab, 7)[0])
        for _ in range(warmup):
            session.run()
        torch.cuda.synchronize()
        assert seqs[0].length == start_ctx
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            session.run()
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / 1e3, session.launches_per_step, start_ctx + steps / 2.0
    finally:
        for s in seqs:
            eng.close_sequence(s)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has")
    ap.add_argument("--sizes", default="0.6b", choices=["0.6b"] + sorted(OTHER_SIZES),
                    help="layer sizes: Qwen3-0.6B (the default run) or those of Qwen3-8B / 14B")
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 / 64 points")
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

    import torch
    from gguf2bin_b200 import kernels
    from gguf2bin_b200.api import LLM
    from gguf2bin_b200.engine import StepEntry
    from gguf2bin_b200.weights import write_random_model

    cfg = dict(QWEN3_0P6B)
    cfg.update(OTHER_SIZES.get(a.sizes, {}))
    full_layers = cfg["num_hidden_layers"]
    if a.layers is None:
        a.layers = full_layers
    cfg["num_hidden_layers"] = a.layers
    name = {"0.6b": "Qwen3-0.6B", "8b": "Qwen3-8B", "14b": "Qwen3-14B"}[a.sizes]
    start_ctx = a.context // 2
    steps = min(a.steps, a.context - start_ctx - 1)
    pk = peaks()
    sizes = model_bytes_and_flops(cfg, a.layers)
    vocab = cfg["vocab_size"]

    with tempfile.TemporaryDirectory(prefix="g2b_bench_") as tmp:
        folder = write_random_model(Path(tmp) / "model", cfg, seed=0, dtype="bfloat16")
        max_batch = 64 if not a.no_points else a.batch
        max_batch = max(max_batch, a.batch)
        llm = LLM(folder, dtype="bfloat16", max_tokens=max_batch * (a.context + 64), max_seqs=max_batch + 1)

        # ---- prefill: one step over a 2,048-token prompt, logits at the last place --------
        prompt = random_prompts(1, PREFILL_TOKENS, vocab, 1)[0]
        pre_ms = []
        for i in range(3 + 3):
            seq = llm.open_sequence()
            llm.engine.cache.reserve(seq, PREFILL_TOKENS)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            llm.step([StepEntry(seq, prompt, (PREFILL_TOKENS - 1,))])
            e1.record()
            torch.cuda.synchronize()
            llm.close_sequence(seq)
            if i >= 3:
                pre_ms.append(e0.elapsed_time(e1))
        pre = statistics.median(pre_ms)
        pre_flops = prefill_flops(cfg, a.layers, PREFILL_TOKENS)
        prefill = dict(value=PREFILL_TOKENS / (pre / 1e3), tokens=PREFILL_TOKENS, ms=pre,
                       frac=pre_flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12))

        # ---- decode, device-timed -----------------------------------------------------------
        clocks = ClockSampler()
        clocks.start()
        launches0 = kernels.launch_count()
        sec, per_step, mean_ctx = decode_device_timed(llm, a.batch, start_ctx, steps, a.warmup, vocab)
        clock_info = clocks.stop()
        value = a.batch * steps / sec
        step_bytes = sizes["weight_bytes"] + a.batch * mean_ctx * sizes["kv_bytes_per_token"]
        achieved = step_bytes / (sec / steps) / 1e9
        roofline = dict(bound="hbm", achieved=achieved, peak=pk["hbm_gbs"], unit="GB/s",
                        frac=achieved / pk["hbm_gbs"], peaks=pk["source"])

        # ---- decode through the Python entry point, host tokens in and out ----------------
        e2e_steps = min(steps, 256)
        prompts = random_prompts(a.batch, start_ctx, vocab, 11)
        llm.generate(prompts[:1], n=4, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                     ignore_eos=True)
        e2e_runs = []                      # three whole calls; the median is reported, all are listed
        for _ in range(3):
            llm.generate(prompts, n=e2e_steps + 1, temperature=0.0, top_k=0, top_p=1.0,
                         repeat_penalty=1.0, ignore_eos=True, max_batch=a.batch)
            acct = llm.last_decode
            e2e_runs.append((acct["tokens"] / acct["seconds"], acct["steps"]))
        e2e_value, e2e_count = sorted(e2e_runs)[1]
        e2e = dict(value=e2e_value, unit="tokens/s", h2d_bytes_per_step=4 * a.batch,
                   d2h_bytes_per_step=4 * a.batch, steps=e2e_count,
                   runs=[round(v, 1) for v, _ in e2e_runs])

        # ---- other batch sizes ------------------------------------------------------------------
        points = {}
        if not a.no_points:
            for b, k in ((1, min(steps, 256)), (64, min(steps, 128))):
                s, _, _ = decode_device_timed(llm, b, start_ctx, k, a.warmup, vocab)
                points[f"decode_b{b}"] = b * k / s

    out = {
        "metric": f"decode tokens/s ({name} sizes, random weights, batch {a.batch}, "
                  f"context {start_ctx}->{a.context})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": a.warmup,
        "ms_per_step": sec / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {"model": f"{name} sizes, random weights", "global_batch": a.batch,
                   "seq_len": a.context, "decode_from": start_ctx, "layers": a.layers,
                   "layers_of_config": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": vocab, "tied": bool(cfg["tie_word_embeddings"]), "parallelism": "none (1 GPU)",
                   "l2": "inputs larger than L2 (weights + cache read every step)",
                   "sampling": "greedy on device"},
        "e2e": e2e, "gpu_launches": per_step * steps, "launches_per_step": per_step,
        "prefill": prefill, "roofline": roofline, "points": points, "clocks": clock_info,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
