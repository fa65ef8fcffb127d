"""A decoder as data: an embedding, a list of layers, the order in which they
run, a final norm and an output head.

The reference's stack is a fixed loop (garuda/src/llama/mod.rs:1092-1095,
:1183-1188); here the order is a list of ``LayerCall``. A layer may be called
twice, and a call may read the cache that an earlier call filled instead of
keeping one of its own. Nothing in this file knows an architecture: an
architecture is a function from its configuration to a ``ModelSpec``
(``garuda_b200/models/llama.py`` is the one there is).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import (PartSpec, TensorSpec, PagedKV, FixedState, LayerCache, build_part,
                          _REGISTRIES)
from ..parts.block import BlockSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order. ``layer`` indexes ``ModelSpec.layers``.
    ``reads_cache_of``: index of an earlier entry of the run order whose cache
    this call reads (it then stores nothing itself)."""
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    width: int
    vocab_size: int
    max_positions: int
    embedding: str                       # tensor name of the [vocab, width] table
    layers: List[BlockSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    head: Optional[str]                  # tensor name of the [vocab, width] head; None: tied
    embedding_init: Tuple = ("normal", 0.02)
    eos_token_ids: Tuple[int, ...] = ()  # generation ends on any of them (config.json may list several)
    # names a model folder may hold although the model reads nothing from them (a tied model's
    # stored copy of its head); anything else the model did not ask for is an error
    ignored_tensors: Tuple[str, ...] = ()

    @property
    def eos_token_id(self) -> Optional[int]:
        return self.eos_token_ids[0] if self.eos_token_ids else None


@dataclass(frozen=True)
class CacheGroup:
    """Calls of the run order whose caches have the same needs and therefore
    share a pool of pages and a block table."""
    need: object                         # PagedKV
    calls: Tuple[int, ...]               # indices into ModelSpec.order (calls that write)


class Decoder:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = [_REGISTRIES["block"][b.arrangement](b) for b in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.ops = None
        self.dtype = None
        # cache needs of the run order
        self.call_need = []
        for i, call in enumerate(spec.order):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {call.layer}, but there are {len(self.blocks)}")
            need = self.blocks[call.layer].mixer.cache_need()
            if call.reads_cache_of is not None:
                src = call.reads_cache_of
                if not 0 <= src < i or spec.order[src].reads_cache_of is not None:
                    raise ValueError(f"run order entry {i} must read the cache of an earlier entry that keeps one")
                if self.call_need[src] != need:
                    raise ValueError(f"run order entry {i} reads a cache of another shape: {self.call_need[src]} vs {need}")
            self.call_need.append(need)
        groups: Dict[object, List[int]] = {}
        self.state_calls: List[int] = []
        for i, (call, need) in enumerate(zip(spec.order, self.call_need)):
            if call.reads_cache_of is not None or need is None:
                continue
            if isinstance(need, PagedKV):
                groups.setdefault(need, []).append(i)
            elif isinstance(need, FixedState):
                self.state_calls.append(i)
            else:
                raise TypeError(f"unknown cache need {need!r}")
        self.cache_groups = [CacheGroup(need, tuple(calls)) for need, calls in groups.items()]

    @property
    def graph_safe(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph: every part says so."""
        return all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe

    # ---- tensors ---------------------------------------------------------
    def expected_tensors(self) -> Dict[str, TensorSpec]:
        s = self.spec
        out = {s.embedding: TensorSpec((s.vocab_size, s.width), init=s.embedding_init)}
        for block in self.blocks:
            for part, prefix in block.parts():
                for local, ts in part.tensors().items():
                    out[prefix + local] = ts
        for local, ts in self.final_norm.tensors().items():
            out[s.final_norm.prefix + local] = ts
        if s.head is not None:
            out[s.head] = TensorSpec((s.vocab_size, s.width), init=s.embedding_init)
        return out

    def load(self, tensors: Dict[str, torch.Tensor], ops, dtype: torch.dtype) -> None:
        """``tensors``: every name of ``expected_tensors()`` on the device."""
        s = self.spec
        self.ops, self.dtype = ops, dtype
        self.embedding = tensors[s.embedding]
        self.head = self.embedding if s.head is None else tensors[s.head]
        for block in self.blocks:
            for part, prefix in block.parts():
                part.load({local: tensors[prefix + local] for local in part.tensors()}, ops, dtype)
        self.final_norm.load({local: tensors[s.final_norm.prefix + local]
                              for local in self.final_norm.tensors()}, ops, dtype)

    # ---- one step ----------------------------------------------------------
    def forward(self, ctx, layer_caches: List[Optional[LayerCache]]) -> torch.Tensor:
        """Runs the batch of ``ctx`` through the run order and returns 32-bit
        logits ``[W, vocab]`` for the batch's ``logit_rows`` only: the final norm
        and the head touch no other row (garuda/src/llama/mod.rs:1110-1113)."""
        b, ops, s = ctx.batch, self.ops, self.spec
        x = ctx.ws.get("residual", (b.num_tokens, s.width), torch.float32)
        ops.embedding(self.embedding, b.token_ids, x)
        # a layer's last product may fold in the first half of the next layer's norm
        pending = None
        for i, call in enumerate(s.order):
            block = self.blocks[call.layer]
            nxt = self.blocks[s.order[i + 1].layer] if i + 1 < len(s.order) else None
            takes = getattr(nxt, "takes_pending_norm", None)
            next_norm = takes(ops) if takes is not None else None
            if pending is not None or next_norm is not None:
                pending = block.forward(ctx, x, layer_caches[i], pending=pending, next_norm=next_norm)
            else:
                pending = block.forward(ctx, x, layer_caches[i])
        w = b.num_logit_rows
        logits = ctx.ws.get("logits", (w, s.vocab_size), torch.float32)
        if w:
            z = self.final_norm.forward(ctx, x, rows=b.logit_rows, out_name="final_normed")
            ops.linear(z, self.head, logits)
        return logits
