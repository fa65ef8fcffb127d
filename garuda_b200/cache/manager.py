"""The paged cache: device memory for the pages, host bookkeeping for who holds which.

Bookkeeping (free lists, block tables, slots) is the C++ ``CacheManager``
(``csrc/host/cache_manager.hpp``). This class adds the device side: for every
group of layer calls with the same needs, a pool ``K`` and ``V`` of shape
``[calls, num_pages, kv_heads, page_size, head_dim]``, and for every call with
state of fixed size an array ``[max_requests, *shape]`` indexed by the request's
slot. The reference keeps both per sequence (garuda/src/cache/mod.rs:221-241,
:610-619, :630-648); here they are pools shared by all requests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..csrc.build import load_host_module
from ..parts.base import LayerCache, PagedKV, FixedState


@dataclass
class CacheConfig:
    page_size: int = 32                 # positions per page (garuda/src/llama/mod.rs:483 uses 32)
    num_pages: Optional[int] = None     # pages per group; None: from max_tokens
    max_tokens: Optional[int] = None    # positions the pool holds per group
    max_requests: int = 4               # request slots (garuda/src/config/mod.rs:166-167)
    max_positions: int = 2048           # positions one request may hold


class PagedCache:
    def __init__(self, model, config: CacheConfig, dtype: torch.dtype, device, allocate: bool = True):
        host = load_host_module()
        self.host_module = host
        self.config = config
        self.model = model
        self.dtype, self.device = dtype, torch.device(device)
        ps = config.page_size
        if config.num_pages is not None:
            pages = int(config.num_pages)
        elif config.max_tokens is not None:
            pages = (int(config.max_tokens) + ps - 1) // ps
        else:
            raise ValueError("the cache needs num_pages or max_tokens")
        self.groups = model.cache_groups
        self.manager = host.CacheManager(
            [host.GroupConfig(pages, g.need.window or 0) for g in self.groups],
            ps, config.max_requests, config.max_positions)
        self.page_size = ps
        self.table_width = self.manager.max_pages_per_request
        # device memory
        self.k_pools: List[torch.Tensor] = []
        self.v_pools: List[torch.Tensor] = []
        self.call_group: Dict[int, tuple] = {}
        for gi, g in enumerate(self.groups):
            shape = (len(g.calls), pages, g.need.kv_heads, ps, g.need.head_dim)
            if allocate:
                self.k_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
                self.v_pools.append(torch.zeros(shape, dtype=dtype, device=self.device))
            for j, call in enumerate(g.calls):
                self.call_group[call] = (gi, j)
        self.states: Dict[int, torch.Tensor] = {}
        for call in model.state_calls:
            need: FixedState = model.call_need[call]
            if allocate:
                self.states[call] = torch.zeros((config.max_requests, *need.shape), dtype=need.dtype,
                                                device=self.device)

    # ---- request lifecycle -------------------------------------------------
    def acquire(self, request: int) -> int:
        """A slot for a new request. Its fixed-size state is zeroed by the step that runs the
        request's first token (``reset_states``), so that it makes no difference who took the
        slot: this call, or a scheduler working on the bookkeeping directly."""
        return self.manager.acquire(request)

    def reset_states(self, slots: Sequence[int]) -> None:
        """Fixed-size state of these slots back to zero, in every layer call that keeps some
        (garuda/src/cache/mod.rs:719-743: a sequence's state starts as zeros)."""
        if not self.states or not slots:
            return
        for s in self.states.values():
            for slot in slots:
                s[slot].zero_()

    def release(self, request: int) -> None:
        self.manager.release(request)

    def bytes_per_position(self) -> int:
        item = self.dtype.itemsize
        return sum(2 * len(g.calls) * g.need.kv_heads * g.need.head_dim * item for g in self.groups)

    # ---- views for a step ------------------------------------------------------
    def layer_caches(self, block_tables: Sequence[torch.Tensor]) -> List[Optional[LayerCache]]:
        """One ``LayerCache`` per entry of the model's run order, over the given
        device block tables (one per group, rows in the batch's request order)."""
        out: List[Optional[LayerCache]] = []
        order = self.model.spec.order
        for i, call in enumerate(order):
            need = self.model.call_need[i]
            src = i if call.reads_cache_of is None else call.reads_cache_of
            if need is None:
                out.append(None)
            elif isinstance(need, PagedKV):
                gi, j = self.call_group[src]
                out.append(LayerCache(need=need, k=self.k_pools[gi][j], v=self.v_pools[gi][j],
                                      block_table=block_tables[gi], page_size=self.page_size,
                                      writes=call.reads_cache_of is None))
            else:
                out.append(LayerCache(need=need, state=self.states[src],
                                      writes=call.reads_cache_of is None))
        return out
