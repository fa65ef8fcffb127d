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
from typing import Sequence

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


class StepRunner:
    """Runs steps. Its host half is the C++ ``StepBuilder`` (``csrc/host/step_batch.hpp``): it checks
    a batch, reserves its pages and writes the arrays that the kernels read into one pinned buffer,
    which goes to the device in one copy."""

    def __init__(self, model, cache: PagedCache, ops, dtype: torch.dtype, device):
        self.model, self.cache, self.ops, self.dtype = model, cache, ops, dtype
        self.device = torch.device(device)
        self.ws = Workspace(self.device)
        self.vocab = model.spec.vocab_size
        self.host = cache.host_module
        self.builder = self.host.StepBuilder(cache.manager, self.vocab)
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
        """The batch for the C++ side and what it reserved: ``(requests, new_lens)``, ``new_lens``
        a list of (request, its length after the step). Raises with nothing changed."""
        try:
            requests = self.host.StepRequests(entries)
            reserved = self.builder.check_and_reserve(requests)
        except self.host.StepError as e:
            raise StepError(str(e)) from None
        # A request that starts at position 0 starts from zeroed fixed-size state, whoever took its
        # slot (this step just now, or a scheduler that admitted it, or readmitted it after it
        # had been preempted) and whoever held the slot before.
        if reserved.starting_slots and self.cache.states:
            self.cache.reset_states(reserved.starting_slots)
        return requests, reserved.new_lens

    # ------------------------------------------------------------------ batch
    def build_batch(self, requests, new_lens) -> StepBatch:
        lay = self.builder.layout(requests)
        pinned = self._stage(lay.words)
        host = pinned.numpy() if pinned is not None else np.empty(lay.words, dtype=np.int32)
        self.builder.fill(requests, new_lens, lay, host)
        if pinned is not None:
            dev = pinned[:lay.words].to(self.device, non_blocking=True)
            if self._staged[self._turn] is None:
                self._staged[self._turn] = torch.cuda.Event()
            self._staged[self._turn].record()
        else:
            dev = torch.from_numpy(host).clone()
        T, R, W, G, width = lay.tokens, lay.rows, lay.wanted, lay.groups, lay.table_width

        def both(at, n):
            return dev[at:at + n], host[at:at + n]

        (token_ids, h_ids), (positions, h_pos), (token_req, h_req) = both(lay.token_ids, T), both(lay.positions, T), both(lay.token_req, T)
        (cu_q, h_cu), (kv_lens, h_kv), (slots, h_slots) = both(lay.cu_q, R + 1), both(lay.kv_lens, R), both(lay.slots, R)
        logit_rows, h_rows = both(lay.logit_rows, W)
        tables = dev[lay.tables:lay.tables + G * R * width].view(G, R, width) if G else None
        return StepBatch(
            num_tokens=T, num_requests=R, token_ids=token_ids, positions=positions, token_req=token_req,
            cu_q=cu_q, kv_lens=kv_lens, slots=slots, block_tables=[tables[g] for g in range(G)],
            logit_rows=logit_rows, num_logit_rows=W, max_q_len=lay.max_q, max_kv_len=lay.max_kv,
            min_q_len=lay.min_q,
            host={"token_ids": h_ids, "positions": h_pos, "token_req": h_req, "cu_q": h_cu, "kv_lens": h_kv,
                  "slots": h_slots, "logit_rows": h_rows, "requests": requests.requests},
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
        requests, new_lens = self._validate_and_reserve(entries)
        if self.graphs is not None and self.graphs.eligible(entries):
            logits = self.graphs.run(entries, requests, new_lens, device_tokens)
            tokens = len(entries)
        else:
            batch = self.build_batch(requests, new_lens)
            ctx = StepContext(batch=batch, ws=self.ws, ops=self.ops, dtype=self.dtype)
            caches = self.cache.layer_caches(batch.block_tables)
            hold = getattr(self.ops, "on_current_stream", None)
            with (hold() if hold is not None else contextlib.nullcontext()):
                logits = self.model.forward(ctx, caches)
            tokens = batch.num_tokens
        self.builder.commit(new_lens)
        self.steps += 1
        self.tokens_run += tokens
        return logits

    def end(self, request: int) -> None:
        """The request is finished: what it holds is given back."""
        self.cache.release(request)
