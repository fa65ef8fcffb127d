"""The flat batch one step runs, and the scratch memory it runs in.

The reference has three call shapes (one sequence with many new tokens, N
sequences with one token each, and a sequential fallback for anything ragged:
garuda/src/llama/mod.rs:1134-1158, :1204-1246). Here there is one: a flat list
of tokens from several requests, each contributing ``q_len >= 1`` consecutive
tokens that start at its current length.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List

import torch


@dataclass
class StepBatch:
    """Device arrays (int32) describing the tokens of one step.

    ``token_ids[T]``, ``positions[T]`` (absolute, 0-based: the request's length
    before the token, as the reference reads it from the cache,
    garuda/src/llama/mod.rs:783), ``token_req[T]`` (row of the request within
    this batch), ``cu_q[R+1]`` (prefix sums of the requests' token counts),
    ``kv_lens[R]`` (length of each request after this step), ``slots[R]`` (state
    slot of each request), ``block_tables[group][R, max_pages]`` and
    ``logit_rows[W]`` (flat token rows whose logits are wanted).
    """
    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_req: torch.Tensor
    cu_q: torch.Tensor
    kv_lens: torch.Tensor
    slots: torch.Tensor
    block_tables: List[torch.Tensor]
    logit_rows: torch.Tensor
    num_logit_rows: int
    max_q_len: int
    max_kv_len: int
    min_q_len: int = 1
    # host copies, for parts written in Python (toy mixers) and for checks
    host: Dict[str, list] = field(default_factory=dict)


class Workspace:
    """Named scratch tensors that live across steps, so that a step allocates
    nothing once sizes have been seen. A buffer grows when a larger shape is
    asked for; a captured CUDA graph owns a workspace of its own so that its
    addresses never change."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._views: Dict[str, tuple] = {}      # name -> (shape, dtype, view): the last view handed out

    def get(self, name: str, shape, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """``zero``: the buffer is zeroed when it is created or grown (not on later calls)."""
        shape = tuple(shape)
        last = self._views.get(name)
        if last is not None and last[0] == shape and last[1] is dtype:
            return last[2]          # the same request as last time (every layer of a step): no new view
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * dtype.itemsize
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < nbytes:
            # 256-byte multiple keeps every view aligned for vector and TMA access
            size = max((nbytes + 255) // 256 * 256, 256)
            make = torch.zeros if zero else torch.empty
            buf = make(size, dtype=torch.uint8, device=self.device)
            self._bufs[name] = buf
        view = buf[:nbytes].view(dtype).view(*shape)
        self._views[name] = (shape, dtype, view)
        return view


@dataclass
class StepContext:
    batch: StepBatch
    ws: Workspace
    ops: object
    dtype: torch.dtype
    # what a step computes once for all its layers (the rotation's cosines and sines), by key
    step_cache: dict = field(default_factory=dict)
    # a part's last product leaves here the norm it folded in (``CudaOps.linear``'s ``emit_norm``)
    pending_norm: object = None
