"""The command line, in the reference's manner.

garuda/src/cli/mod.rs:10-44: ``garuda [-c|--config FILE] [subcommand]`` with the
configuration file before the subcommand, defaults when the file does not exist
(garuda/src/main.rs:30-36), ``benchmark -i/--iterations -t/--tokens`` and
``inspect FILE``. The reference's ``serve`` (its HTTP servers) is not part of
this engine; ``generate``, ``init`` and ``replay`` are this engine's own.
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="garuda", description="B200-native inference engine for dense Llama decoders")
    ap.add_argument("-c", "--config", default="config.toml", metavar="FILE",
                    help="configuration file; defaults are used if it does not exist")
    ap.add_argument("--plugin", action="append", default=[], metavar="MODULE",
                    help="import this module first (it registers an architecture or parts of its own); "
                         "also [model] plugins in the configuration file")
    sub = ap.add_subparsers(dest="command")
    g = sub.add_parser("generate", help="generate from token ids")
    g.add_argument("--prompt-ids", required=True, action="append",
                   help="comma-separated token ids; repeat for several prompts")
    g.add_argument("--max-tokens", type=int)
    g.add_argument("--temperature", type=float)
    g.add_argument("--top-k", type=int)
    g.add_argument("--top-p", type=float)
    g.add_argument("--seed", type=int)
    b = sub.add_parser("benchmark", help="measure startup, time to first token, per-token latency, tokens/s")
    b.add_argument("-i", "--iterations", type=int, default=64)
    b.add_argument("-t", "--tokens", type=int, default=32, help="tokens to generate per iteration")
    b.add_argument("--prompt-len", type=int, default=60, help="tokens of the fixed random prompt")
    b.add_argument("--batch", default="1", metavar="N[,N...]",
                   help="requests generating together; a list measures each in turn, e.g. 1,8,64")
    i = sub.add_parser("inspect", help="print the configuration and tensors of a model folder")
    i.add_argument("folder")
    n = sub.add_parser("init", help="random-weights mode: write a model folder from a config.json and a seed")
    n.add_argument("folder")
    n.add_argument("--config-json", required=True, help="the architecture's config.json to use")
    n.add_argument("--seed", type=int, default=0)
    n.add_argument("--store-dtype", choices=["float32", "bfloat16"], default="bfloat16")
    r = sub.add_parser("replay", help="feed the steps of a trace through the step function and write logits")
    r.add_argument("trace", help="file of steps, one JSON object a line; - reads standard input")
    r.add_argument("out", help="folder for the logits files <step>.f32")
    r.add_argument("--max-tokens", type=int, default=0,
                   help="tokens the cache pool is made for (default: the configuration file's)")
    sub.add_parser("serve", help="not part of this engine")
    return ap


def _sampling(cfg, args):
    from .sampling.params import SamplingParams
    s = cfg.sampling
    pick = lambda a, b: b if a is None else a
    return SamplingParams(temperature=pick(getattr(args, "temperature", None), s.temperature),
                          top_p=pick(getattr(args, "top_p", None), s.top_p),
                          top_k=pick(getattr(args, "top_k", None), s.top_k),
                          max_tokens=pick(getattr(args, "max_tokens", None), s.max_tokens),
                          seed=getattr(args, "seed", None))


def cmd_generate(cfg, args) -> int:
    from .engine.engine import Engine
    engine = Engine.from_config(cfg)
    prompts = [[int(x) for x in p.split(",") if x.strip()] for p in args.prompt_ids]
    for r in engine.generate(prompts, _sampling(cfg, args)):
        print(json.dumps({"tokens": r.tokens, "finish_reason": r.finish_reason, "error": r.error}))
    return 0


def cmd_benchmark(cfg, args) -> int:
    """garuda/src/benchmark/mod.rs:17-188: one fixed prompt, a warm-up run, then
    ``iterations`` runs of ``tokens`` tokens; startup, mean time to first token,
    per-token latency and tokens per second, all measured. ``--batch`` runs that
    many copies of the prompt together (the reference measures one sequence)."""
    import numpy as np
    from .engine.engine import Engine
    from .sampling.params import SamplingParams
    try:
        batches = [int(b) for b in str(args.batch).split(",") if b.strip()]
    except ValueError:
        batches = []
    if not batches or min(batches) < 1:
        print(f"error: --batch wants positive numbers, got {args.batch!r}", file=sys.stderr)
        return 2
    print("=== garuda_b200 benchmark ===")
    t0 = time.perf_counter()
    engine = Engine.from_config(cfg, max_concurrent=max(cfg.server.max_concurrent, max(batches)))
    startup = time.perf_counter() - t0
    spec = engine.model.spec
    print(f"model: {cfg.model.path} ({spec.architecture}: {len(spec.order)} layer calls, width {spec.width}, "
          f"vocabulary {spec.vocab_size})")
    print(f"startup                {startup:12.2f} s")
    rng = np.random.default_rng(0xBEEF)
    n = max(min(args.prompt_len, engine.max_context - args.tokens - 1), 1)
    prompt = rng.integers(0, spec.vocab_size, n).tolist()
    params = SamplingParams(temperature=cfg.sampling.temperature, top_p=cfg.sampling.top_p,
                            top_k=cfg.sampling.top_k, max_tokens=args.tokens, seed=0xBEEF)
    for batch in batches:
        prompts = [prompt] * batch
        engine.generate(prompts, params)                      # warm-up
        total = first = 0.0
        generated = 0
        stops = {"eos": 0, "length": 0}
        for _ in range(max(args.iterations, 1)):
            seen = []
            start = time.perf_counter()
            res = engine.generate(prompts, params, on_token=lambda i, t: seen.append(time.perf_counter()))
            total += time.perf_counter() - start
            first += (seen[0] - start) if seen else 0.0
            generated += sum(len(r.tokens) for r in res)
            for r in res:
                stops["eos" if r.finish_reason == "eos" else "length"] += 1
        print(f"--- batch {batch}")
        print(f"prompt                 {n:12d} tokens x {batch}")
        print(f"generated              {generated:12d} tokens over {args.iterations} runs")
        print(f"time to first token    {first / max(args.iterations, 1) * 1e3:12.2f} ms")
        print(f"per-token latency      {total / max(generated, 1) * 1e3:12.3f} ms")
        print(f"throughput             {generated / total:12.1f} tok/s")
        print(f"stopped on eos/length  {stops['eos']:5d} / {stops['length']}")
    st = engine.stats()
    print(f"steps / preemptions    {st['steps']:5d} / {st['preemptions']}")
    return 0


def cmd_replay(cfg, args) -> int:
    """Trace replay (``garuda_b200/engine/replay.py``) on the model and the settings of the
    configuration file. The closest thing in the reference are its tests that feed a prompt in
    differently cut pieces (garuda/src/llama/mod.rs:1556-1612)."""
    from .engine.engine import Engine
    from .engine.replay import replay, _say_done
    extra = {"kv_tokens": args.max_tokens} if args.max_tokens else {}
    engine = Engine.from_config(cfg, **extra)
    if args.trace == "-":
        replay(engine, sys.stdin, args.out, report=_say_done)
    else:
        with open(args.trace, "r", encoding="utf-8") as f:
            replay(engine, f, args.out, report=_say_done)
    return 0


def cmd_inspect(args) -> int:
    """garuda/src/main.rs:56-148: what the file holds, and whether it will load."""
    from .config.model_config import read_config_json, ConfigError
    from .config.registry import build_model
    from .weights.safetensors_io import SafetensorsFolder, SafetensorsError
    from .weights.loader import check_folder
    try:
        raw = read_config_json(args.folder)
        cfg, model = build_model(raw)
    except ConfigError as e:
        print(f"config.json: {e}\nloadable: no")
        return 1
    print(f"architecture: {model.spec.architecture}")
    import dataclasses
    as_dict = cfg.to_dict() if hasattr(cfg, "to_dict") else (
        dataclasses.asdict(cfg) if dataclasses.is_dataclass(cfg) else dict(vars(cfg)))
    for k, v in as_dict.items():
        if k not in ("architectures",):
            print(f"  {k} = {v}")
    try:
        folder = SafetensorsFolder(args.folder)
    except SafetensorsError as e:
        print(f"weights: {e}\nloadable: no")
        return 1
    total = 0
    for name in sorted(folder.names()):
        e = folder.entries[name]
        n = 1
        for s in e.shape:
            n *= s
        total += n
        print(f"  {name:60s} {e.dtype:5s} {list(e.shape)}")
    print(f"tensors: {len(folder.entries)}, parameters: {total}")
    missing, unexpected, wrong, other = check_folder(model, folder)
    if missing or unexpected or wrong or other:
        for label, items in (("missing", missing), ("unexpected", unexpected),
                             ("wrong shape", [w[0] for w in wrong]), ("other", other)):
            if items:
                print(f"{label}: {', '.join(items)}")
        print("loadable: no")
        return 1
    print("loadable: yes")
    return 0


def cmd_init(args) -> int:
    import torch
    from .weights.random_init import write_random_model
    with open(args.config_json, "r", encoding="utf-8") as f:
        config = json.load(f)
    dt = torch.float32 if args.store_dtype == "float32" else torch.bfloat16
    write_random_model(args.folder, config, args.seed, store_dtype=dt)
    print(f"wrote {args.folder}/config.json and model.safetensors (seed {args.seed})")
    return 0


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    from .config.engine_config import EngineConfig
    from .config.model_config import ConfigError
    from .config.registry import load_plugins
    try:
        cfg = EngineConfig.load_or_default(args.config) if args.command not in ("init",) else None
        load_plugins(list(args.plugin) + (list(cfg.model.plugins) if cfg is not None else []))
    except ConfigError as e:
        if args.command != "inspect":
            print(f"error: {e}", file=sys.stderr)
            return 1
        cfg = None
        load_plugins(args.plugin)
    if args.command == "inspect":
        return cmd_inspect(args)
    if args.command == "init":
        return cmd_init(args)
    if args.command in (None, "serve"):
        print("garuda_b200 has no server: use `generate`, `benchmark`, `replay`, `inspect` or `init`",
              file=sys.stderr)
        return 2
    return {"generate": cmd_generate, "benchmark": cmd_benchmark, "replay": cmd_replay}[args.command](cfg, args)


if __name__ == "__main__":
    sys.exit(main())
