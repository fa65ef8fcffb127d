"""The step function: one batch of (request, its next tokens) in, logits at the
wanted places out.

The reference's contract for a forward call (garuda/src/core/mod.rs:232-261):
consume only positions not seen yet, advance every layer by one position per
token, fail with an error and not a panic, be deterministic; and nothing is
half-applied: a batch is checked before any cache is touched
(garuda/src/llama/mod.rs:1160-1172, :1061-1067). The same holds here, for a
batch that may mix portions of prompts with single decoded tokens, cut anywhere.
A step runs only the tokens it is given; everything earlier comes from the cache.
"""
from __future__ import annotations

import contextlib

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import PagedCache
from .batch import StepBatch, StepContext, Workspace


class StepError(ValueError):
    """A batch that was refused; no request and no page has changed."""


@dataclass
class StepEntry:
    request: int                      # the caller's id of the request
    tokens: Sequence[int]             # its next tokens, in order
    want: Sequence[int] = field(default_factory=tuple)   # places among them whose logits are wanted


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


class StepRunner:
    def __init__(self, model, cache: PagedCache, ops, dtype: torch.dtype, device):
        self.model, self.cache, self.ops, self.dtype = model, cache, ops, dtype
        self.device = torch.device(device)
        self.ws = Workspace(self.device)
        self.vocab = model.spec.vocab_size
        self.steps = 0
        self.tokens_run = 0
        self.graphs = None        # DecodeGraphs, when decode steps are replayed from CUDA graphs
        # pinned staging for the batch's arrays: two buffers in turn, each with an event that tells
        # when the copy that last read it has run (pinning memory anew for every step costs far more
        # than the copy)
        self._staging = [None, None]
        self._staged = [None, None]
        self._turn = 0

    # ------------------------------------------------------------------ checks
    def _validate_and_reserve(self, entries: Sequence[StepEntry]):
        mgr = self.cache.manager
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        wants = []
        fresh = []
        starting = []          # requests whose first token this step runs
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request} brings no tokens")
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab:
                    raise StepError(f"token {t} of request {e.request} is outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not 0 <= int(w) < n:
                    raise StepError(f"request {e.request} wants logits at place {w} of {n} tokens")
            known = mgr.known(e.request)
            old = mgr.length(e.request) if known else 0
            if old + n > mgr.max_positions:
                raise StepError(f"{n} tokens do not fit the {mgr.max_positions}-position context "
                                f"({old} used) of request {e.request}")
            if not known:
                fresh.append(e.request)
            if old == 0:
                starting.append(e.request)
            wants.append((e.request, old + n))
        if len(fresh) > mgr.free_slots:
            raise StepError(f"{len(fresh)} new requests but only {mgr.free_slots} request slots are free")
        for r in fresh:
            self.cache.acquire(r)
        try:
            if not mgr.can_reserve(wants):
                need = [mgr.pages_needed(r, n) for r, n in wants]
                total = [sum(x[g] for x in need) for g in range(mgr.num_groups)]
                free = [mgr.free_pages(g) for g in range(mgr.num_groups)]
                raise self.cache.host_module.OutOfPages(
                    f"the step needs {total} pages per group but only {free} are free")
            for r, n in wants:
                mgr.reserve(r, n)
        except Exception:
            for r in fresh:
                mgr.release(r)
            raise
        # A request that starts at position 0 starts from zeroed fixed-size state, whoever took its
        # slot (this runner just now, or a scheduler that admitted it, or readmitted it after it
        # had been preempted) and whoever held the slot before.
        if starting and self.cache.states:
            self.cache.reset_states([mgr.slot(r) for r in starting])
        return wants

    # ------------------------------------------------------------------ batch
    def build_batch(self, entries: Sequence[StepEntry], new_lens) -> StepBatch:
        mgr = self.cache.manager
        R = len(entries)
        T = sum(len(e.tokens) for e in entries)
        W = sum(len(e.want) for e in entries)
        G, width = mgr.num_groups, self.cache.table_width
        offs = {}
        cursor = 0
        for name, n in (("token_ids", T), ("positions", T), ("token_req", T), ("cu_q", R + 1),
                        ("kv_lens", R), ("slots", R), ("logit_rows", max(W, 1)),
                        ("tables", G * R * width)):
            offs[name] = (cursor, n)
            cursor += _align(n)
        pinned = self._stage(cursor)
        host = pinned.numpy()[:cursor] if pinned is not None else np.empty(cursor, dtype=np.int32)

        def view(name):
            o, n = offs[name]
            return host[o:o + n]

        token_ids, positions, token_req = view("token_ids"), view("positions"), view("token_req")
        cu_q, kv_lens, slots, logit_rows = view("cu_q"), view("kv_lens"), view("slots"), view("logit_rows")
        logit_rows[:] = 0
        t = w = 0
        cu_q[0] = 0
        max_q = max_kv = 0
        min_q = 1 << 30
        for i, (e, (_, new_len)) in enumerate(zip(entries, new_lens)):
            n = len(e.tokens)
            start = new_len - n
            token_ids[t:t + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[t:t + n] = np.arange(start, new_len, dtype=np.int32)
            token_req[t:t + n] = i
            for place in e.want:
                logit_rows[w] = t + int(place)
                w += 1
            t += n
            cu_q[i + 1] = t
            kv_lens[i] = new_len
            slots[i] = mgr.slot(e.request)
            max_q, max_kv, min_q = max(max_q, n), max(max_kv, new_len), min(min_q, n)
        tables = view("tables").reshape(G, R, width) if G else None
        if G:
            mgr.fill_block_tables([e.request for e in entries], tables)

        if pinned is not None:
            dev = pinned[:cursor].to(self.device, non_blocking=True)
            if self._staged[self._turn] is None:
                self._staged[self._turn] = torch.cuda.Event()
            self._staged[self._turn].record()
        else:
            dev = torch.from_numpy(host).clone()

        def dview(name):
            o, n = offs[name]
            return dev[o:o + n]

        dtables = [dview("tables").view(G, R, width)[g] for g in range(G)] if G else []
        return StepBatch(
            num_tokens=T, num_requests=R, token_ids=dview("token_ids"), positions=dview("positions"),
            token_req=dview("token_req"), cu_q=dview("cu_q"), kv_lens=dview("kv_lens"),
            slots=dview("slots"), block_tables=dtables, logit_rows=dview("logit_rows")[:W],
            num_logit_rows=W, max_q_len=max_q, max_kv_len=max_kv, min_q_len=min_q,
            host={"token_ids": token_ids, "positions": positions, "token_req": token_req, "cu_q": cu_q,
                  "kv_lens": kv_lens, "slots": slots, "logit_rows": logit_rows[:W],
                  "requests": [e.request for e in entries]},
        )

    def _stage(self, n: int):
        """A pinned int32 buffer of at least ``n`` entries that no copy in flight still reads, or
        None on a machine without a device."""
        if self.device.type != "cuda":
            return None
        self._turn ^= 1
        t = self._turn
        if self._staged[t] is not None:
            self._staged[t].synchronize()
        buf = self._staging[t]
        if buf is None or buf.numel() < n:
            size = 1024
            while size < n:
                size *= 2
            buf = self._staging[t] = torch.empty(size, dtype=torch.int32).pin_memory()
        return buf

    # ------------------------------------------------------------------ run
    def run(self, entries: Sequence[StepEntry], device_tokens=None) -> torch.Tensor:
        """Logits ``[W, vocab]`` (float32, on the device) at the wanted places, in
        the order of the entries and of their ``want``. Valid until the next step.
        ``device_tokens``: for a step of single tokens that are still on their way from
        the step in front (int32 on the device, in the entries' order; the entries' own
        tokens are placeholders then). Only decode steps replayed from graphs take it."""
        if device_tokens is not None and not (self.graphs is not None and self.graphs.eligible(entries)):
            raise StepError("tokens on the device are taken by graph-replayed decode steps only")
        new_lens = self._validate_and_reserve(entries)
        if self.graphs is not None and self.graphs.eligible(entries):
            logits = self.graphs.run(entries, new_lens, device_tokens)
            tokens = len(entries)
        else:
            batch = self.build_batch(entries, new_lens)
            ctx = StepContext(batch=batch, ws=self.ws, ops=self.ops, dtype=self.dtype)
            caches = self.cache.layer_caches(batch.block_tables)
            hold = getattr(self.ops, "on_current_stream", None)
            with (hold() if hold is not None else contextlib.nullcontext()):
                logits = self.model.forward(ctx, caches)
            tokens = batch.num_tokens
        mgr = self.cache.manager
        for r, n in new_lens:
            mgr.commit(r, n)
        self.steps += 1
        self.tokens_run += tokens
        return logits

    def end(self, request: int) -> None:
        """The request is finished: what it holds is given back."""
        self.cache.release(request)
