#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step: every live request advances by one token. The default
run has the layer sizes of TinyLlama-1.1B with random weights, 8 requests and a
context of 2,048 tokens. Times are taken with CUDA events on the launching
stream, after warm-up, with a synchronize on both sides. Nothing flushes L2
between steps: a decode step reads every weight once (over 2 GB), far more than
L2 holds. The end-to-end figure goes through ``Engine.generate`` with token ids
coming from and going back to the host every step.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

TINYLLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=2048,
                 num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
                 intermediate_size=5632, vocab_size=32000, rope_theta=10000.0, rms_norm_eps=1e-5,
                 tie_word_embeddings=False, max_position_embeddings=2048)
FULL_LAYERS = 22
CONTEXT = 2048
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_PEAKS["hbm_gbs"], FALLBACK_PEAKS["bf16_tflops"], "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """Call at the start and at the end of the timed region."""
        self.marks = getattr(self, "marks", []) + [time.time()]

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        marks = getattr(self, "marks", [])
        lo, hi = (marks[0], marks[-1]) if len(marks) >= 2 else (0.0, float("inf"))

        def collect(inside):
            sm, mx, reasons = [], [], set()
            for when, line in self.lines:
                # a sample is printed up to one period after it was taken
                if inside and not (lo <= when <= hi + 0.06):
                    continue
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, v in zip(names, parts[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            return sorted(sm), mx, reasons

        sm, mx, reasons = collect(True)
        window = "timed region"
        if not sm:       # the region was shorter than the sampling period: the samples around it
            sm, mx, reasons = collect(False)
            window = "decode phase around the timed region"
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "window": window}


def model_bytes_and_flops(cfg, layers, batch, kv_len, itemsize=2):
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = d * (q + 2 * kv) + q * d + 3 * d * ff
    weight_bytes = (layers * per_layer + V * d) * itemsize          # every matrix once; norms are negligible
    cache_bytes = batch * kv_len * layers * 2 * kv * itemsize
    return per_layer, weight_bytes, cache_bytes


def run_ours(args) -> dict:
    import numpy as np
    import torch
    from garuda_b200 import Engine, SamplingParams, StepEntry
    from garuda_b200.weights import write_random_model

    layers = args.layers
    cfg = dict(TINYLLAMA, num_hidden_layers=layers)
    hbm_peak, tflops_peak, peak_kind = peaks()
    K, W = args.steps, args.warmup
    tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    try:
        t0 = time.time()
        write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
        print(f"[bench] wrote random weights in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        engine = Engine(tmp, dtype="bfloat16", context=CONTEXT, page_size=32, kv_tokens=64 * CONTEXT,
                        max_concurrent=64, queue_capacity=256, max_batch_tokens=PREFILL_TOKENS,
                        prefill_chunk=PREFILL_TOKENS, ignore_eos=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    runner, ops = engine.runner, engine.ops
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)

    if args.only:
        return run_one_phase(args, engine, cfg, rng)

    # ---------------------------------------------------------------- prefill, 2048 tokens in one step
    toks = rng.integers(0, V, PREFILL_TOKENS).tolist()
    times = []
    for i in range(3 + 5):
        s, e = ev(), ev()
        torch.cuda.synchronize()
        s.record()
        runner.run([StepEntry(1000 + i, toks, [PREFILL_TOKENS - 1])])
        e.record()
        torch.cuda.synchronize()
        runner.end(1000 + i)
        if i >= 3:
            times.append(s.elapsed_time(e))
    prefill_ms = sorted(times)[len(times) // 2]
    per_layer, _, _ = model_bytes_and_flops(cfg, layers, 1, 0)
    T = PREFILL_TOKENS
    flops = 2 * T * layers * per_layer + 2 * V * cfg["hidden_size"] \
        + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2)
    prefill = {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (tflops_peak * 1e12), 4)}

    # ---------------------------------------------------------------- decode
    def decode(batch, steps, warmup, sample_clocks=False):
        """Requests prefilled so that the last timed step reaches the full context."""
        start_len = CONTEXT - steps - warmup
        ids = list(range(batch))
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.start()          # early: nvidia-smi takes a moment to print its first sample
        for r in ids:
            runner.run([StepEntry(r, rng.integers(0, V, start_len).tolist(), [])])
        feed = rng.integers(0, V, (steps + warmup, batch))
        out = torch.empty(batch, dtype=torch.int32, device=engine.device)

        def one(i):
            logits = runner.run([StepEntry(r, [int(feed[i, j])], [0]) for j, r in enumerate(ids)])
            ops.argmax(logits, out)

        for i in range(warmup):
            one(i)
        launches0 = ops.launches
        s, e = ev(), ev()
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
        s.record()
        for i in range(warmup, warmup + steps):
            one(i)
        e.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
            time.sleep(0.12)         # let the sample taken at the end be printed
        clocks = sampler.stop() if sampler else None
        ms = s.elapsed_time(e) / steps
        launches = ops.launches - launches0 + runner.graphs.launches_replayed(batch) * steps
        for r in ids:
            runner.end(r)
        mean_kv = CONTEXT - steps / 2
        return ms, clocks, launches, mean_kv

    ms8, clocks, launches, mean_kv = decode(8, K, W, sample_clocks=True)
    _, wbytes, cbytes = model_bytes_and_flops(cfg, layers, 8, mean_kv)
    achieved = (wbytes + cbytes) / (ms8 * 1e-3) / 1e9
    ms1, _, _, _ = decode(1, min(K, 32), W)
    ms64, _, _, _ = decode(64, min(K, 32), W)
    ops.tc.check_errors()

    # ---------------------------------------------------------------- end to end through Engine.generate
    prompts = [rng.integers(0, V, CONTEXT - K - W - 1).tolist() for _ in range(8)]
    stamps = []
    engine.warm_up()      # graphs of the smaller batches, which the run's last rounds use as requests end
    engine.generate(prompts, SamplingParams.greedy(max_tokens=K + W), on_token=lambda i, t: stamps.append(time.perf_counter()))
    torch.cuda.synchronize()
    # the first W rounds of 8 tokens are warm-up (they also hold the prefill); the rest is timed
    timed = stamps[8 * W - 1:]
    e2e_value = (len(timed) - 1) / (timed[-1] - timed[0]) if len(timed) > 1 else 0.0
    cap = runner.graphs.graphs.get(8)
    h2d = int(cap.pinned.numel() * 4) if cap is not None else 0
    # the same with sampled requests (the reference's default temperature, top-k and top-p), as a point
    stamps_s = []
    engine.generate(prompts, SamplingParams(temperature=0.8, top_k=40, top_p=0.95, max_tokens=K + W, seed=1),
                    on_token=lambda i, t: stamps_s.append(time.perf_counter()))
    torch.cuda.synchronize()
    timed_s = stamps_s[8 * W - 1:]
    e2e_sampled = (len(timed_s) - 1) / (timed_s[-1] - timed_s[0]) if len(timed_s) > 1 else 0.0

    return {
        "metric": "decode tok/s at batch 8, context 2048 (TinyLlama-1.1B shape, random weights)",
        "value": round(8 / ms8 * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
        "config": {"model": "TinyLlama-1.1B shape", "layers": layers, "layers_full": FULL_LAYERS,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied": False, "global_batch": 8, "seq_len": CONTEXT,
                   "context_at_first_timed_step": CONTEXT - K, "page_size": 32, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": "inputs larger than L2 (weights 2.07 GB per step)",
                   "peaks": peak_kind},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 8 * 4},
        "gpu_launches": int(launches),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4)},
        "points": {"decode_b1": round(1 / ms1 * 1e3, 1), "decode_b64": round(64 / ms64 * 1e3, 1),
                   "e2e_sampled_b8": round(e2e_sampled, 1)},
        "clocks": clocks,
    }


def run_one_phase(args, engine, cfg, rng) -> dict:
    """One phase only, for profiling: `--only prefill` runs a 2,048-token prompt `steps` times,
    `--only decode` prefills `--batch` requests and runs `steps` decode steps. Prints times, not the
    benchmark record."""
    import torch
    from garuda_b200 import StepEntry
    runner, V = engine.runner, cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    times = []
    if args.only == "prefill":
        toks = rng.integers(0, V, PREFILL_TOKENS).tolist()
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(i, toks, [PREFILL_TOKENS - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.end(i)
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
    else:
        ids = list(range(args.batch))
        start_len = CONTEXT - args.steps - args.warmup
        for r in ids:
            runner.run([StepEntry(r, rng.integers(0, V, start_len).tolist(), [])])
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(r, [int(rng.integers(0, V))], [0]) for r in ids])
            e.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
    engine.ops.tc.check_errors()
    return {"only": args.only, "batch": args.batch, "layers": args.layers, "ms": [round(t, 4) for t in times]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", choices=["prefill", "decode"], help="run one phase only (for profiling)")
    ap.add_argument("--batch", type=int, default=8, help="requests of the decode phase with --only decode")
    ap.add_argument("--layers", type=int, default=FULL_LAYERS,
                    help="fewer layers than the configuration has (reported beside the full number)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "hanumanit/garuda is a Rust crate without a Python package; no cargo/rustc here, "
                          "its dependencies are not vendored and there is no network, so it cannot be built"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine does not run on {args.gpus} GPUs")
        return 2
    args.warmup = max(args.warmup, 3)
    args.steps = max(1, min(args.steps, 512))
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
