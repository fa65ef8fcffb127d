"""Decode steps replayed from captured CUDA graphs.

A decode step is a few hundred short kernels; launched one by one from the
host they cost more than they run. A step in which every request brings one
token is therefore captured once per batch-size bucket and replayed: the
kernels read the batch's token ids, positions, lengths and block tables from
fixed device buffers that are refilled before every replay. Rows beyond the
live requests are padding: a request of one token whose block table holds no
page, which the kernels skip.
"""
from __future__ import annotations

import gc
from typing import Dict

import torch

from .batch import StepBatch, StepContext, Workspace


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class _Captured:
    def __init__(self, graph, logits, host, dev, layout):
        self.graph, self.logits, self.host, self.dev, self.layout = graph, logits, host, dev, layout


class DecodeGraphs:
    def __init__(self, runner, max_requests: int):
        self.runner = runner
        self.max_bucket = _bucket(max_requests)
        self.graphs: Dict[int, _Captured] = {}
        self.replays = 0

    def eligible(self, entries) -> bool:
        """A step of single tokens, of a model whose every part may be captured (``graph_safe``)."""
        return (self.runner.model.graph_safe and len(entries) <= self.max_bucket
                and all(len(e.tokens) == 1 for e in entries))

    # ------------------------------------------------------------------ arrays
    def _batch(self, cap: _Captured, B: int) -> StepBatch:
        mgr = self.runner.cache.manager
        lay = cap.layout
        G, width = lay.groups, lay.table_width

        def dview(at, n):
            return cap.dev[at:at + n]

        tables = [dview(lay.tables, G * B * width).view(G, B, width)[g] for g in range(G)] if G else []
        return StepBatch(num_tokens=B, num_requests=B, token_ids=dview(lay.token_ids, B),
                         positions=dview(lay.positions, B), token_req=dview(lay.token_req, B),
                         cu_q=dview(lay.cu_q, B + 1), kv_lens=dview(lay.kv_lens, B), slots=dview(lay.slots, B),
                         block_tables=tables, logit_rows=dview(lay.logit_rows, B), num_logit_rows=B,
                         max_q_len=1, max_kv_len=mgr.max_positions, host={})

    # ------------------------------------------------------------------ capture
    def _capture(self, B: int) -> _Captured:
        r = self.runner
        # the arrays of a step of B single tokens, as the C++ step builder lays them out and fills them
        layout = r.builder.decode_layout(B)
        size = layout.words
        # Two pinned staging buffers in turn, each with an event that tells when its copy to the device
        # has run: a caller that does not read a step's logits (a prompt's unwanted tokens, a timing
        # loop) comes back before the copy of the step in front has happened, and must not overwrite
        # what that copy will read.
        staging = [torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(2)]
        host = staging[0]
        dev = torch.zeros(size, dtype=torch.int32, device=r.device)
        cap = _Captured(None, None, host.numpy(), dev, layout)
        cap.pinned = host
        cap.staging, cap.copied, cap.turn = staging, [None, None], 0
        r.builder.fill_decode(r.host.StepRequests([]), [], layout, cap.host)
        dev.copy_(host, non_blocking=True)
        batch = self._batch(cap, B)
        ws = Workspace(r.device)
        ctx = StepContext(batch=batch, ws=ws, ops=r.ops, dtype=r.dtype)
        caches = r.cache.layer_caches(batch.block_tables)
        # once outside the capture: tables and scratch that are made on first use. The kernel set notes
        # meanwhile which weights the step streams, in order, and tells every product of the captured
        # run what comes behind it.
        tc = getattr(r.ops, "tc", None)
        if tc is not None:
            tc.record_streams()
        r.model.forward(ctx, caches)
        torch.cuda.synchronize(r.device)
        if tc is not None:
            tc.hint_streams()
        graph = torch.cuda.CUDAGraph()
        before = getattr(r.ops, "launches", 0)
        # a context of its own: what the run above made "once per step" (the rotation's table) must be
        # made inside the graph too, or a replay would rotate by the angles of the capture's positions
        ctx = StepContext(batch=batch, ws=ws, ops=r.ops, dtype=r.dtype)
        # No garbage collection in the middle of the capture: garbage that holds device memory or
        # graphs (an engine that was dropped earlier) would be freed there, and freeing device memory
        # invalidates a capture. Other threads may use the device meanwhile (thread_local).
        collecting = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, capture_error_mode="thread_local"), r.ops.on_current_stream():
                logits = r.model.forward(ctx, caches)
        finally:
            if collecting:
                gc.enable()
            if tc is not None:
                tc.forget_streams()
        cap.launches = getattr(r.ops, "launches", 0) - before      # kernels one replay runs
        if hasattr(r.ops, "launches"):
            r.ops.launches = before
        cap.graph, cap.logits, cap.ws = graph, logits, ws
        return cap

    def warm(self) -> None:
        """Captures every bucket now (a few milliseconds each) rather than at the first step
        that needs it."""
        B = 1
        while B <= self.max_bucket:
            if B not in self.graphs:
                self.graphs[B] = self._capture(B)
            B *= 2

    def launches_replayed(self, num_requests: int) -> int:
        """Kernels that one replay for this many requests launches."""
        cap = self.graphs.get(_bucket(num_requests))
        return cap.launches if cap is not None else 0

    # ------------------------------------------------------------------ run
    def run(self, entries, requests, new_lens, device_tokens=None) -> torch.Tensor:
        """``requests``: the entries as the step builder holds them. ``device_tokens``: int32 on the
        device, the entries' tokens in their order, for a step whose tokens the host does not know
        yet (they come from the step in front)."""
        B = _bucket(len(entries))
        cap = self.graphs.get(B)
        if cap is None:
            cap = self.graphs[B] = self._capture(B)
        cap.turn ^= 1
        cap.pinned = cap.staging[cap.turn]
        cap.host = cap.pinned.numpy()
        if cap.copied[cap.turn] is not None:
            cap.copied[cap.turn].synchronize()      # the copy that last read this buffer has run
        self.runner.builder.fill_decode(requests, new_lens, cap.layout, cap.host)
        cap.dev.copy_(cap.pinned, non_blocking=True)
        if cap.copied[cap.turn] is None:
            cap.copied[cap.turn] = torch.cuda.Event()
        cap.copied[cap.turn].record()
        if device_tokens is not None:
            o = cap.layout.token_ids
            cap.dev[o:o + len(entries)].copy_(device_tokens[:len(entries)])
        cap.graph.replay()
        self.replays += 1
        rows = [i for i, e in enumerate(entries) if len(e.want)]
        if len(rows) == len(entries):
            return cap.logits[:len(entries)]
        return cap.logits[torch.tensor(rows, dtype=torch.long, device=cap.logits.device)]
