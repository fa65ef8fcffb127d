"""Trace replay: feed given token ids through a model step by step, write logits.

It samples nothing and has no forward pass, cache or loader of its own: it
drives an ``Engine``'s step function, the one generation uses. The closest
thing in the reference are its unit tests that feed a prompt in differently cut
pieces and compare logits (garuda/src/llama/mod.rs:1556-1612, :1640-1715).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` holds the logits
at the wanted places (order of the entries, then of ``want``) as little-endian
float32 ``[wanted, vocab]``. After every step a line ``done <step>`` is printed
and flushed.

Three ways in: ``bin/trace_run`` (steps on standard input), ``garuda replay
TRACE OUT`` (a file, or ``-`` for standard input) and ``Engine.replay``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Iterable


def replay(engine, lines: Iterable[str], out_dir: str, report=None) -> int:
    """Runs the steps that ``lines`` describe through ``engine.step`` and writes the logits
    files into ``out_dir``. ``report(step)`` is called after every step. Returns the number of
    steps run. Request ids of the trace are the trace's own (any JSON string or number); a
    request that is named in ``end`` gives back what it holds."""
    from .step import StepEntry
    os.makedirs(out_dir, exist_ok=True)
    ids = {}
    next_id = 1 << 40          # out of the way of ids that a scheduler hands out
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            if e["id"] not in ids:
                ids[e["id"]] = next_id
                next_id += 1
            entries.append(StepEntry(ids[e["id"]], e["tokens"], e.get("want", [])))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                arr = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        engine.check_errors()
        for name in rec.get("end", []):
            if name in ids:
                if engine.cache.manager.known(ids[name]):
                    engine.runner.end(ids[name])
                del ids[name]
        steps += 1
        if report is not None:
            report(step)
    return steps


def _say_done(step) -> None:
    print(f"done {step}", flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder the logits files go to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=32)
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--plugin", action="append", default=[], metavar="MODULE",
                    help="import this module first (it registers an architecture or parts of its own)")
    args = ap.parse_args(argv)

    from ..config.registry import load_plugins
    from .engine import Engine

    load_plugins(args.plugin)
    engine = Engine(args.model, dtype=args.dtype, page_size=args.page_size, kv_tokens=args.max_tokens,
                    max_concurrent=args.max_requests, cuda_graphs=not args.no_graphs)
    replay(engine, sys.stdin, args.out, report=_say_done)
    return 0


if __name__ == "__main__":
    sys.exit(main())
