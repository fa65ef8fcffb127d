"""The Python entry point: a model folder in, generated tokens out.

The reference's programmatic surface is ``Engine::build`` (garuda/src/server/mod.rs:48-54,
:343-479: read the configuration, open the checkpoint, dispatch on its
architecture, size the cache, build the runtime) followed by
``Scheduler::submit`` (garuda/src/scheduler/mod.rs:258-303) or
``InferenceRuntime::start`` / ``next_token`` (garuda/src/runtime/mod.rs:560, :698).
``Engine`` here does the first, ``generate`` the second: it submits every
prompt to the scheduler and runs mixed steps until all have finished.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional, Sequence, Union

import torch

from ..cache.manager import PagedCache, CacheConfig
from ..config.engine_config import EngineConfig, parse_size
from ..config.model_config import ConfigError, read_config_json
from ..config.registry import build_model
from ..csrc.build import load_host_module
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_weights
from .step import StepRunner, StepEntry, StepError

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class GenerationResult:
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""          # "length" | "context_full" | "eos" | "error"
    error: Optional[str] = None      # with "error": the message ("cancelled", "timeout", a failed step's, ...)


@dataclass
class StreamEvent:
    """One event of a request's output (garuda/src/scheduler/mod.rs:67-71)."""
    index: int                       # which prompt of the call
    kind: str                        # "token" | "done" | "error"
    token: Optional[int] = None
    detail: Optional[str] = None     # done: "length" | "context_full" | "eos"; error: the message
    request: int = -1                # the scheduler's id of the request (``Engine.scheduler.cancel``)


class Engine:
    def __init__(self, model_dir: str, dtype="bfloat16", *, context: Optional[int] = None,
                 sliding_window: int = 0, page_size: int = 32, kv_tokens: Optional[int] = None,
                 kv_cache_bytes: Optional[int] = None, max_concurrent: int = 4,
                 queue_capacity: int = 256, max_batch_tokens: int = 2048, prefill_chunk: int = 2048,
                 cuda_graphs: bool = True, lookahead: bool = True, device: int = 0, ignore_eos: bool = False,
                 eos_token_id: Union[None, int, Sequence[int]] = None,
                 request_timeout: Optional[float] = None, paced_prefill: bool = False, ops=None):
        """``request_timeout``: seconds from its submission after which a request, waiting or
        running, ends with the error "timeout" (garuda/src/scheduler/mod.rs:520); None: no limit.
        ``paced_prefill``: while something is decoding, prompts go in by portions that cost about
        one decode step, sized from the measured times of the steps (garuda/src/scheduler/mod.rs:305-370)."""
        if dtype not in _DTYPES:
            raise ConfigError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}")
        self.dtype = _DTYPES[dtype]
        self.model_dir = model_dir
        if request_timeout is not None and not request_timeout > 0:
            raise ConfigError(f"request_timeout must be positive, got {request_timeout!r}")
        self.request_timeout = None if request_timeout is None else float(request_timeout)
        config_dict = read_config_json(model_dir)
        if sliding_window:
            config_dict = dict(config_dict, sliding_window=int(sliding_window))
        if ops is None:
            from ..kernels.ops import CudaOps
            self.device = torch.device(f"cuda:{device}")
            torch.cuda.set_device(self.device)
            # the 32-bit path never touches a tensor core: true 32-bit multiply-adds throughout
            ops = CudaOps(self.device, tensor_cores=self.dtype == torch.bfloat16)
        else:
            self.device = torch.device(getattr(ops, "device", "cpu"))
        self.ops = ops
        self.config, self.model = build_model(config_dict)
        load_weights(self.model, model_dir, ops, self.dtype, self.device)

        spec = self.model.spec
        self.max_context = min(int(context), spec.max_positions) if context else spec.max_positions
        if self.max_context < 2:
            raise ConfigError("the context must hold at least 2 tokens")
        probe = PagedCache(self.model, CacheConfig(page_size=page_size, num_pages=0,
                                                   max_requests=max_concurrent,
                                                   max_positions=self.max_context),
                           self.dtype, self.device, allocate=False)
        if kv_tokens:
            tokens = int(kv_tokens)
        elif kv_cache_bytes:
            per_position = max(probe.bytes_per_position(), 1)
            tokens = int(kv_cache_bytes) // per_position
        else:
            tokens = max_concurrent * self.max_context
        pages = max((tokens + page_size - 1) // page_size, 1)
        self.cache = PagedCache(self.model, CacheConfig(page_size=page_size, num_pages=pages,
                                                        max_requests=max_concurrent,
                                                        max_positions=self.max_context),
                                self.dtype, self.device)
        self.runner = StepRunner(self.model, self.cache, ops, self.dtype, self.device)
        self.sampler = Sampler(ops, self.device)
        host = load_host_module()
        self._host = host
        sc = host.SchedulerConfig()
        sc.max_concurrent = max_concurrent
        sc.queue_capacity = queue_capacity
        sc.max_batch_tokens = max_batch_tokens
        sc.prefill_chunk = prefill_chunk
        sc.max_context = self.max_context
        sc.vocab_size = spec.vocab_size
        # generation ends on any of the architecture's end tokens (config.json may list several),
        # or on those given here in their place
        if eos_token_id is None:
            eos = tuple(spec.eos_token_ids)
        elif isinstance(eos_token_id, int):
            eos = (int(eos_token_id),)
        else:
            eos = tuple(int(t) for t in eos_token_id)
        sc.eos_token_ids = list(eos)
        sc.ignore_eos = bool(ignore_eos)
        sc.paced_prefill = bool(paced_prefill)
        self.paced_prefill = bool(paced_prefill)
        self.scheduler = host.Scheduler(sc, self.cache.manager)
        self.cuda_graphs = bool(cuda_graphs) and self.device.type == "cuda"
        # launch the next greedy decode step before this step's tokens have reached the host
        self.lookahead = bool(lookahead) and self.cuda_graphs
        if self.cuda_graphs:
            from .graph import DecodeGraphs
            self.runner.graphs = DecodeGraphs(self.runner, max_concurrent)

    @classmethod
    def from_config(cls, cfg: EngineConfig, **overrides) -> "Engine":
        kv_bytes = parse_size(cfg.memory.kv_cache)
        kwargs = dict(
            dtype=cfg.model.dtype, context=cfg.model.context, sliding_window=cfg.model.sliding_window,
            page_size=cfg.memory.page_size, kv_tokens=cfg.memory.kv_tokens or None,
            kv_cache_bytes=kv_bytes or None, max_concurrent=cfg.server.max_concurrent,
            queue_capacity=cfg.server.queue_capacity, max_batch_tokens=cfg.runtime.max_batch_tokens,
            prefill_chunk=cfg.runtime.prefill_chunk, cuda_graphs=cfg.runtime.cuda_graphs,
            lookahead=cfg.runtime.lookahead, paced_prefill=cfg.runtime.paced_prefill,
            request_timeout=cfg.server.request_timeout_secs,
            device=cfg.runtime.device)
        kwargs.update(overrides)
        return cls(cfg.model.path, **kwargs)

    # ------------------------------------------------------------------ raw step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """One step of the step function; see ``StepRunner.run``."""
        return self.runner.run(entries)

    def check_errors(self) -> None:
        """Raises ``KernelError`` if a kernel of a step that has finished gave up on a bounded wait
        (its results are then not to be trusted). Free of copies and synchronisation: it reads a
        word of pinned host memory that such a kernel writes; call it after waiting for a step's
        results. ``generate`` and ``replay`` do."""
        failed = getattr(self.ops, "failed_wait", None)
        if failed is not None and failed():
            self.ops.tc.check_errors()       # synchronises, clears, raises with the code's meaning

    def replay(self, trace, out_dir: str, report=None) -> int:
        """Trace replay through this engine's step function: ``trace`` is a path of a file of
        steps (one JSON object a line, see ``garuda_b200/engine/replay.py``) or an iterable of such
        lines; logits of the wanted places go to ``out_dir/<step>.f32``. Returns the number of steps."""
        from .replay import replay
        if isinstance(trace, (str, bytes)):
            with open(trace, "r", encoding="utf-8") as f:
                return replay(self, f, out_dir, report)
        return replay(self, trace, out_dir, report)

    def warm_up(self) -> None:
        """Captures the decode step's graphs for every batch size now, so that no request
        waits for a capture later (a capture takes some milliseconds, once per bucket)."""
        if self.runner.graphs is not None:
            self.runner.graphs.warm()

    # ------------------------------------------------------------------ generate
    def _host_params(self, p: SamplingParams):
        p.validate()
        return self._host.SamplingParams(temperature=p.temperature, top_p=p.top_p, top_k=p.top_k,
                                         max_tokens=p.max_tokens, seed=p.seed)

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[None, SamplingParams, Sequence[SamplingParams]] = None,
                 on_token=None, timeout: Optional[float] = None,
                 priority: Union[int, Sequence[int]] = 0) -> List[GenerationResult]:
        """Generate for every prompt (lists of token ids), batching them
        continuously. ``sampling``: one ``SamplingParams`` for all, or one per
        prompt. ``on_token(index, token)`` is called as tokens arrive; if it returns False, that
        request is cancelled (it ends with the error "cancelled" before the next step). ``timeout``: seconds
        after its submission at which a request ends with the error "timeout", checked between
        steps (default: the engine's ``request_timeout``). ``priority``: one for all or one per
        prompt; among waiting requests the higher goes first, equal ones in order of arrival
        (garuda/src/scheduler/mod.rs:138-148)."""
        results = [GenerationResult() for _ in prompts]
        for ev in self.stream(prompts, sampling, timeout=timeout, priority=priority):
            r = results[ev.index]
            if ev.kind == "token":
                r.tokens.append(ev.token)
                # a callback that answers False has gone: its request is cancelled between steps, as
                # a closed stream is in the reference (garuda/src/scheduler/mod.rs:616-621)
                if on_token is not None and on_token(ev.index, ev.token) is False:
                    self.scheduler.cancel(ev.request)
            elif ev.kind == "done":
                r.finish_reason = ev.detail
            else:
                r.finish_reason, r.error = "error", ev.detail
        return results

    def stream(self, prompts: Sequence[Sequence[int]],
               sampling: Union[None, SamplingParams, Sequence[SamplingParams]] = None,
               timeout: Optional[float] = None, priority: Union[int, Sequence[int]] = 0) -> Iterator[StreamEvent]:
        """The events of ``generate`` as they happen, in the reference's manner
        (garuda/src/scheduler/mod.rs:67-71): for every prompt its tokens, then one ``done`` (with
        the reason) or ``error`` (with the message). Closing the iterator before its end, or
        dropping it, cancels what is still running (a dropped handle cancels: :92-109)."""
        if timeout is None:
            timeout = self.request_timeout
        elif not timeout > 0:
            raise ConfigError(f"timeout must be positive, got {timeout!r}")
        if sampling is None:
            sampling = SamplingParams()
        if isinstance(sampling, SamplingParams):
            sampling = [sampling] * len(prompts)
        if len(sampling) != len(prompts):
            raise ConfigError(f"{len(sampling)} sampling settings for {len(prompts)} prompts")
        priorities = [int(p) for p in priority] if hasattr(priority, "__iter__") else [int(priority)] * len(prompts)
        if len(priorities) != len(prompts):
            raise ConfigError(f"{len(priorities)} priorities for {len(prompts)} prompts")
        return self._events(prompts, sampling, float(timeout or 0.0), priorities)

    def _events(self, prompts, sampling, timeout: float, priorities):
        index_of: Dict[int, int] = {}
        pending = list(range(len(prompts)))
        sched = self.scheduler
        kinds = self._host.EventKind

        def told(events):
            for ev in events:
                i = index_of.get(ev.id)
                if i is None:
                    continue
                if ev.kind == kinds.Token:
                    yield StreamEvent(i, "token", token=ev.token, request=ev.id)
                else:
                    del index_of[ev.id]
                    yield StreamEvent(i, "done" if ev.kind == kinds.Done else "error", detail=ev.detail,
                                      request=ev.id)

        ahead = None      # (ids, Pending): a decode step launched before its plan was made
        try:
            while pending or index_of:
                while pending:
                    i = pending[0]
                    try:
                        rid = sched.submit(list(map(int, prompts[i])), self._host_params(sampling[i]),
                                           priorities[i], timeout)
                    except self._host.Busy:
                        break      # the queue is full: run steps, then submit the rest
                    except (self._host.SchedulerError, ConfigError) as e:
                        pending.pop(0)
                        yield StreamEvent(i, "error", detail=str(e))
                        continue
                    index_of[rid] = i
                    pending.pop(0)
                if not index_of:
                    continue
                plan = sched.plan()
                yield from told(plan.events)
                if not plan.entries:
                    ahead = None
                    continue
                started = time.perf_counter()
                try:
                    collect, ahead = self._run_plan(plan, ahead)
                    tokens = collect()
                except Exception as exc:     # the step failed as a whole: its requests end with the error
                    ahead = None
                    yield from told(sched.fail(plan, f"{type(exc).__name__}: {exc}"))
                    continue
                # what the step took, for the pacing of prompt portions (with steps launched ahead: the
                # wait for this step's tokens, about one step in the steady state)
                elapsed = time.perf_counter() - started if self.paced_prefill else -1.0
                yield from told(sched.complete(plan, tokens, elapsed))
        finally:
            # left before the end: nobody reads what is still running, so it is cancelled, and the
            # scheduler gives back what it held (the next plan does that; it runs no step)
            if index_of:
                for rid in index_of:
                    sched.cancel(rid)
                sched.plan()

    def _run_plan(self, plan, ahead):
        """Runs a plan's entries and starts drawing their tokens. Returns ``(collect,
        ahead)``: ``collect()`` waits for the tokens (one per sampled entry, in the plan's
        order); ``ahead`` is a decode step for the same requests, launched at once with
        its tokens read on the device from this step's draw, or None.

        Launching ahead keeps the GPU busy while the host waits for this step's tokens,
        lets the scheduler finish and plan, and prepares the next launch. A step ahead
        is only launched for decode steps, whose next entries are known but for the
        tokens (a sampled entry's uniform draw is the next of its request's generator,
        which the scheduler lets us look at). When the plan to come turns out different (a request has finished
        or was preempted, another has joined), the rows of the step ahead that still
        fit are used and the plan's other entries run as a step of their own; a row
        for a request that is gone is dropped (what it wrote to the cache lies in pages
        that are given back with the request)."""
        entries = list(plan.entries)
        have = {}
        if ahead is not None:
            gone = set(plan.preempted)
            have = {rid: k for k, rid in enumerate(ahead[0]) if rid not in gone}
        matched = [e for e in entries if e.sample and len(e.tokens) == 1 and e.id in have]
        for e in matched:       # a row of the step ahead was drawn with the uniform that the plan now brings
            if e.temperature != 0.0 and e.u != ahead[2][e.id]:
                raise RuntimeError(f"request {e.id}: the step launched ahead drew with {ahead[2][e.id]}, the plan brings {e.u}")
        taken = {e.id for e in matched}
        rest = [e for e in entries if e.id not in taken]
        fresh = None
        if rest:
            logits = self.runner.run([StepEntry(e.id, e.tokens, (len(e.tokens) - 1,) if e.sample else ())
                                      for e in rest])
            rows = [e for e in rest if e.sample]
            fresh = self.sampler.launch(logits, [e.temperature for e in rows], [e.top_k for e in rows],
                                        [e.top_p for e in rows], [e.u for e in rows])
        # where each sampled entry's token will be: ("ahead", row) or ("fresh", row)
        where, k = [], 0
        for e in entries:
            if not e.sample:
                continue
            if e.id in taken:
                where.append((0, have[e.id]))
            else:
                where.append((1, k))
                k += 1

        nxt = None
        if (self.lookahead and self.runner.graphs is not None and self.model.graph_safe
                and all(e.sample and len(e.tokens) == 1 for e in entries)):
            try:
                if not rest and [w[1] for w in where] == list(range(len(ahead[0]))):
                    dev_tokens = ahead[1].tokens
                elif not matched:
                    dev_tokens = fresh.tokens
                else:
                    parts = [(ahead[1].tokens if src == 0 else fresh.tokens)[row:row + 1] for src, row in where]
                    dev_tokens = torch.cat(parts)
                step = [StepEntry(e.id, (0,), (0,)) for e in entries]
                logits = self.runner.run(step, device_tokens=dev_tokens)
                # a sampled row's uniform draw comes from the request's generator in its fixed order, so
                # the draw of the step ahead is known now (the scheduler hands it out again with the plan)
                us = [0.0 if e.temperature == 0.0 else self.scheduler.peek_uniform(e.id) for e in entries]
                nxt = ([e.id for e in entries],
                       self.sampler.launch(logits, [e.temperature for e in entries], [e.top_k for e in entries],
                                           [e.top_p for e in entries], us),
                       dict(zip((e.id for e in entries), us)))
            except (StepError, self._host.CacheError):
                nxt = None        # no room (pages, context) to run ahead: the scheduler decides next time

        def collect():
            a = self.sampler.result(ahead[1]) if matched else []
            f = self.sampler.result(fresh) if fresh is not None else []
            self.check_errors()      # the step's kernels have finished: did one of them give up on a wait?
            return [(a if src == 0 else f)[row] for src, row in where]

        return collect, nxt

    def stats(self) -> dict:
        s = self.scheduler.stats()
        m = self.cache.manager
        out = {k: getattr(s, k) for k in ("submitted", "completed", "cancelled", "timed_out", "failed", "rejected_busy",
                                          "preemptions", "steps", "tokens_fed", "tokens_generated",
                                          "running", "queued")}
        out["pages_free"] = [m.free_pages(g) for g in range(m.num_groups)]
        out["pages_total"] = [m.total_pages(g) for g in range(m.num_groups)]
        out["pages_reused"] = m.pages_reused
        out["engine_steps"] = self.runner.steps
        return out
