#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

    python bench.py --shape tinyllama|llama2-7b|llama3-8b [--layers L]

A step is one decode step: every live request advances by one token. The default
run has the layer sizes of TinyLlama-1.1B with random weights, 8 requests and a
context of 2,048 tokens; ``--shape`` chooses another of the reference's published
shapes. Times are taken with CUDA events on the launching stream, after warm-up,
with a synchronize on both sides of the timed region and an event after every
step inside it (so that the median step is known beside the mean). Nothing
flushes L2 between steps: a decode step reads every weight once (gigabytes), far
more than L2 holds. The end-to-end figure goes through ``Engine.generate`` with
token ids coming from and going back to the host every step. Fractions are
given against the peaks measured on this pool (``MEASURED_PEAKS.json``) and
against the nominal ones. The reference itself runs on the CPU only and cannot be
built here; what stands in for its "CPU seconds" is the plain implementation of
the tests on the smallest published configuration.
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

LLAMA = dict(architectures=["LlamaForCausalLM"], model_type="llama", rms_norm_eps=1e-5, tie_word_embeddings=False)
# layer sizes of the reference's published configurations; `context`: the benchmark's context length
SHAPES = {
    "tinyllama": dict(name="TinyLlama-1.1B shape", context=2048, layers_default=22, config=dict(
        LLAMA, hidden_size=2048, num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
        intermediate_size=5632, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=2048)),
    # the larger shapes run with a quarter of their layers by default (the layers are alike; writing and
    # loading 13 to 15 GB of random weights would take minutes): `config` names both numbers
    "llama2-7b": dict(name="Llama-2-7B shape", context=4096, layers_default=8, config=dict(
        LLAMA, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32, head_dim=128,
        intermediate_size=11008, vocab_size=32000, rope_theta=10000.0, max_position_embeddings=4096)),
    "llama3-8b": dict(name="Llama-3-8B shape", context=8192, layers_default=8, config=dict(
        LLAMA, hidden_size=4096, num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=8192)),
}
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops": 2250.0}     # HBM3e of the HGX B200; dense bfloat16 tensor rate


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
                                          "--format=csv,noheader,nounits", "-lms", "20"],
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

    shape = SHAPES[args.shape]
    full_layers = shape["config"]["num_hidden_layers"]
    layers = args.layers or shape["layers_default"]
    context = shape["context"]
    cfg = dict(shape["config"], num_hidden_layers=layers)
    hbm_peak, tflops_peak, peak_kind = peaks()
    K, W = args.steps, args.warmup
    batch = args.batch
    # the cache: 64 requests at a context of at most 2,048 (the 64-request point), or the headline's
    # requests at the shape's own context, whichever is more
    b64_context = min(context, 2048)
    kv_tokens = max(64 * b64_context, batch * context) + 64 * 32
    tmp = tempfile.mkdtemp(prefix="garuda_bench_", dir="/dev/shm" if os.path.isdir("/dev/shm") else None)
    try:
        t0 = time.time()
        write_random_model(tmp, cfg, seed=0, store_dtype=torch.bfloat16)
        print(f"[bench] wrote random weights in {time.time() - t0:.0f} s", file=sys.stderr, flush=True)
        engine = Engine(tmp, dtype="bfloat16", context=context, page_size=32, kv_tokens=kv_tokens,
                        max_concurrent=64, queue_capacity=256, max_batch_tokens=PREFILL_TOKENS,
                        prefill_chunk=PREFILL_TOKENS, ignore_eos=True)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    runner, ops = engine.runner, engine.ops
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)

    if args.only:
        return run_one_phase(args, engine, cfg, rng, context)

    # ---------------------------------------------------------------- prompts in one step
    def prefill(tokens, at=0):
        """Median milliseconds of a step of `tokens` prompt tokens that start at position `at`."""
        toks = rng.integers(0, V, tokens).tolist()
        before = rng.integers(0, V, at).tolist() if at else None
        times = []
        for i in range(3 + 5):
            rid = 1000 + i
            if before:
                for lo in range(0, at, PREFILL_TOKENS):
                    runner.run([StepEntry(rid, before[lo:lo + PREFILL_TOKENS], [])])
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(rid, toks, [tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.end(rid)
            if i >= 3:
                times.append(s.elapsed_time(e))
        return sorted(times)[len(times) // 2]

    per_layer, _, _ = model_bytes_and_flops(cfg, layers, 1, 0)

    def prefill_flops(T, at=0):
        keys = T * at + T * (T + 1) // 2
        return 2 * T * layers * per_layer + 2 * V * cfg["hidden_size"] \
            + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * keys

    def prefill_record(T, ms, at=0):
        rate = prefill_flops(T, at) / (ms * 1e-3)
        return {"value": round(T / ms * 1e3, 1), "tokens": T, "ms": round(ms, 3),
                "frac": round(rate / (tflops_peak * 1e12), 4), "tflops": round(rate / 1e12, 1),
                "frac_nominal": round(rate / (NOMINAL["bf16_tflops"] * 1e12), 4)}

    prefill_ms = prefill(PREFILL_TOKENS)
    prefill_rec = prefill_record(PREFILL_TOKENS, prefill_ms)
    points = {}
    if context > PREFILL_TOKENS:
        # the last 2,048 tokens of a prompt as long as the shape's own context
        ms = prefill(PREFILL_TOKENS, at=context - PREFILL_TOKENS)
        points[f"prefill_last_2048_of_{context}_frac"] = prefill_record(PREFILL_TOKENS, ms, context - PREFILL_TOKENS)["frac"]
        points[f"prefill_last_2048_of_{context}_ms"] = round(ms, 3)
    points["prefill_512_ms"] = round(prefill(512), 3)

    # ---------------------------------------------------------------- decode
    def decode(nreq, steps, warmup, ctx_len, sample_clocks=False, beside=0):
        """Requests prefilled so that the last timed step reaches the full context. `beside`: every
        step also carries a prompt portion of that many tokens of another request (a mixed step)."""
        start_len = ctx_len - steps - warmup
        ids = list(range(nreq))
        sampler = ClockSampler() if sample_clocks else None
        if sampler:
            sampler.start()          # early: nvidia-smi takes a moment to print its first sample
        for r in ids:
            toks = rng.integers(0, V, start_len).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.run([StepEntry(r, toks[lo:lo + PREFILL_TOKENS], [])])
        feed = rng.integers(0, V, (steps + warmup, nreq))
        extra = rng.integers(0, V, beside * (steps + warmup)).tolist() if beside else None
        out = torch.empty(nreq, dtype=torch.int32, device=engine.device)

        def one(i):
            entries = [StepEntry(r, [int(feed[i, j])], [0]) for j, r in enumerate(ids)]
            if beside:
                entries.append(StepEntry(9000, extra[i * beside:(i + 1) * beside], []))
            logits = runner.run(entries)
            ops.argmax(logits, out)
            if beside:
                runner.end(9000)     # the next step's portion starts a prompt again

        for i in range(warmup):
            one(i)
        launches0 = ops.launches
        marks = [ev() for _ in range(steps + 1)]
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
        marks[0].record()
        for i in range(warmup, warmup + steps):
            one(i)
            marks[i - warmup + 1].record()
        torch.cuda.synchronize()
        if sampler:
            sampler.mark()
            time.sleep(0.06)         # let the sample taken at the end be printed
        clocks = sampler.stop() if sampler else None
        ms = marks[0].elapsed_time(marks[-1]) / steps
        each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
        launches = ops.launches - launches0 + runner.graphs.launches_replayed(nreq) * (0 if beside else steps)
        for r in ids:
            runner.end(r)
        return ms, each[len(each) // 2], clocks, launches, ctx_len - steps / 2

    ms_b, med_b, clocks, launches, mean_kv = decode(batch, K, W, context, sample_clocks=True)
    _, wbytes, cbytes = model_bytes_and_flops(cfg, layers, batch, mean_kv)
    achieved = (wbytes + cbytes) / (ms_b * 1e-3) / 1e9
    side = min(K, 64)

    def frac_of(nreq, ms, ctx_len):
        _, wb, cb = model_bytes_and_flops(cfg, layers, nreq, ctx_len - side / 2)
        return round((wb + cb) / (ms * 1e-3) / 1e9 / hbm_peak, 4)

    ms1, _, _, _, _ = decode(1, side, W, context)
    ms64, _, _, _, _ = decode(64, side, W, b64_context)
    mixed_ms, _, _, _, _ = decode(8, min(K, 8), W, min(context, 2048), beside=504)
    ops.tc.check_errors()
    points.update({"decode_b1": round(1 / ms1 * 1e3, 1), "decode_b64": round(64 / ms64 * 1e3, 1),
                   "decode_b1_ms": round(ms1, 4), "decode_b64_ms": round(ms64, 4),
                   "decode_b1_hbm_frac": frac_of(1, ms1, context), "decode_b64_hbm_frac": frac_of(64, ms64, b64_context),
                   "decode_b64_context": b64_context, "mixed_step_8_decode_504_prompt_ms": round(mixed_ms, 3)})

    # ---------------------------------------------------------------- end to end through Engine.generate
    prompts = [rng.integers(0, V, context - K - W - 1).tolist() for _ in range(batch)]

    def steady_rate(stamps):
        """Tokens a second while all requests decode together: from the moment the last request to
        start has had its W warm-up tokens (with long prompts the first requests decode beside the
        others' prompt portions for a while) to the moment the first request ends."""
        per = {}
        for i, when in stamps:
            per.setdefault(i, []).append(when)
        if len(per) < batch or min(len(v) for v in per.values()) <= W:
            return 0.0
        t0 = max(v[W - 1] for v in per.values())
        t1 = min(v[-1] for v in per.values())
        inside = sorted(when for _, when in stamps if t0 <= when <= t1)
        return (len(inside) - 1) / (inside[-1] - inside[0]) if len(inside) > 1 and inside[-1] > inside[0] else 0.0

    stamps = []
    engine.warm_up()      # graphs of the smaller batches, which the run's last rounds use as requests end
    engine.generate(prompts, SamplingParams.greedy(max_tokens=K + W), on_token=lambda i, t: stamps.append((i, time.perf_counter())))
    torch.cuda.synchronize()
    e2e_value = steady_rate(stamps)
    cap = runner.graphs.graphs.get(batch)
    h2d = int(cap.pinned.numel() * 4) if cap is not None else 0
    # the same with sampled requests (the reference's default temperature, top-k and top-p), as a point
    stamps_s = []
    engine.generate(prompts, SamplingParams(temperature=0.8, top_k=40, top_p=0.95, max_tokens=K + W, seed=1),
                    on_token=lambda i, t: stamps_s.append((i, time.perf_counter())))
    torch.cuda.synchronize()
    points["e2e_sampled"] = round(steady_rate(stamps_s), 1)
    engine.check_errors()

    return {
        "metric": f"decode tok/s at batch {batch}, context {context} ({shape['name']}, random weights)",
        "value": round(batch / ms_b * 1e3, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_b, 4), "ms_per_step_median": round(med_b, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0, 0.02) and uniform random token ids",
        "config": {"model": shape["name"], "layers": layers, "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "q_heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": V, "rope_theta": cfg["rope_theta"],
                   "rms_norm_eps": cfg["rms_norm_eps"], "tied": False, "global_batch": batch, "seq_len": context,
                   "context_at_first_timed_step": context - K, "page_size": 32, "parallelism": "single GPU",
                   "cuda_graphs": True, "l2": f"inputs larger than L2 (weights {wbytes / 1e9:.2f} GB per step)",
                   "peaks": peak_kind},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": batch * 4},
        "gpu_launches": int(launches),
        "prefill": prefill_rec,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s",
                     "frac": round(achieved / hbm_peak, 4), "peak_nominal": NOMINAL["hbm_gbs"],
                     "frac_nominal": round(achieved / NOMINAL["hbm_gbs"], 4)},
        "points": points,
        "cpu_reference": cpu_reference_seconds(),
        "clocks": clocks,
    }


def cpu_reference_seconds() -> dict:
    """The reference is a CPU engine; it cannot be built here, so the nearest thing to its time is
    the plain implementation of the tests (its formulas, numpy, 32-bit, no cache) on the smallest of
    its published configurations: three prompts of up to 48 tokens, whole, and 16 greedy tokens each."""
    try:
        import numpy as np
        from garuda_b200.weights.random_init import random_weights
        from tests.plain import llama_plain
        cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                   num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
                   rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=128)
        w = {k: v.float().numpy() for k, v in random_weights(cfg, 0).items()}
        rng = np.random.default_rng(0)
        prompts = [rng.integers(0, 256, n).tolist() for n in (1, 24, 48)]
        t0 = time.perf_counter()
        for p in prompts:
            llama_plain.forward(cfg, w, p)
        t1 = time.perf_counter()
        for p in prompts:
            llama_plain.greedy_generate(cfg, w, p, 16)
        t2 = time.perf_counter()
        return {"what": "plain numpy implementation, Tiny A (2 layers, hidden 64), 3 prompts of 1/24/48 tokens",
                "prefill_seconds": round(t1 - t0, 4), "generate_16_tokens_each_seconds": round(t2 - t1, 4)}
    except Exception as e:      # the tests' plain model is not part of an installed package
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_one_phase(args, engine, cfg, rng, context) -> dict:
    """One phase only, for profiling: `--only prefill` runs a 2,048-token prompt `steps` times,
    `--only decode` prefills `--batch` requests and runs `steps` decode steps, `--only attention` runs
    the attention kernel alone on the last `--tokens` tokens of one request of `--context` (random
    queries, keys and values in the engine's own cache layout). Prints times, not the benchmark
    record."""
    import torch
    from garuda_b200 import StepEntry
    runner, V = engine.runner, cfg["vocab_size"]
    ev = lambda: torch.cuda.Event(enable_timing=True)
    times = []
    if args.only == "attention":
        T, ctx_len, page = args.tokens, max(args.context or args.tokens, args.tokens), 32
        Hq, Hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        npages = (ctx_len + page - 1) // page
        dev, ops = engine.device, engine.ops
        k, v = (torch.randn(npages + 1, Hkv, page, hd, device=dev).bfloat16() for _ in range(2))
        q = torch.randn(T, Hq, hd, device=dev).bfloat16()
        out = torch.zeros(T, Hq * hd, device=dev, dtype=torch.bfloat16)
        table = torch.arange(npages, dtype=torch.int32, device=dev).view(1, npages)
        cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
        kvl = torch.tensor([ctx_len], dtype=torch.int32, device=dev)
        treq = torch.zeros(T, dtype=torch.int32, device=dev)
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            ops.paged_attention(q, k, v, table, cu, kvl, treq, out, hd ** -0.5, 0, page, 1, T, ctx_len, min_q_len=T)
            e.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
        ops.tc.check_errors()
        ms = sorted(times)[len(times) // 2]
        flops = 4.0 * Hq * hd * (T * (ctx_len - T) + T * (T + 1) / 2)
        return {"only": "attention", "shape": args.shape, "tokens": T, "context": ctx_len, "heads": Hq, "kv_heads": Hkv,
                "head_dim": hd, "us": round(ms * 1e3, 1), "tflops_causal": round(flops / ms / 1e9, 1)}
    if args.only == "prefill":
        toks = rng.integers(0, V, args.tokens).tolist()
        for i in range(args.warmup + args.steps):
            s, e = ev(), ev()
            torch.cuda.synchronize()
            s.record()
            runner.run([StepEntry(i, toks, [args.tokens - 1])])
            e.record()
            torch.cuda.synchronize()
            runner.end(i)
            if i >= args.warmup:
                times.append(s.elapsed_time(e))
    else:
        ids = list(range(args.batch))
        ctx_len = min(context, args.context or context)
        start_len = ctx_len - args.steps - args.warmup
        for r in ids:
            toks = rng.integers(0, V, start_len).tolist()
            for lo in range(0, start_len, PREFILL_TOKENS):
                runner.run([StepEntry(r, toks[lo:lo + PREFILL_TOKENS], [])])
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
    return {"only": args.only, "shape": args.shape, "batch": args.batch, "layers": cfg["num_hidden_layers"],
            "ms": [round(t, 4) for t in times]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="tinyllama", choices=sorted(SHAPES),
                    help="layer sizes: one of the reference's published configurations")
    ap.add_argument("--only", choices=["prefill", "decode", "attention"], help="run one phase only (for profiling)")
    ap.add_argument("--batch", type=int, default=8, help="requests of the timed decode steps")
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="prompt tokens with --only prefill")
    ap.add_argument("--context", type=int, default=0, help="context reached with --only decode (default: the shape's); keys with --only attention")
    ap.add_argument("--layers", type=int, default=0,
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
    if not 1 <= args.batch <= 64:
        print("bench.py: --batch must be 1 to 64")
        return 2
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
