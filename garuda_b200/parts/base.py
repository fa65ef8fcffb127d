"""Interfaces of the parts a decoder is put together from, and their registries.

A part is a mixer (attention here), a feed-forward, a norm or a position
encoding. Each takes its sizes and constants as constructor parameters, names
the tensors it needs, and knows nothing about the model it sits in: the same
class serves any layer of any architecture, and a model may name different
parts in different layers. The reference keeps these as methods of one struct
(garuda/src/llama/mod.rs:733-1020); here each is a class chosen by name.

A new part is added by subclassing the matching base class and registering it
with ``register_mixer`` / ``register_feed_forward`` / ``register_norm`` /
``register_position_encoding``; a model's layer list then refers to it by that
name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Optional, Tuple

import torch


# --------------------------------------------------------------------------
# what a part asks of the loader and of the cache
# --------------------------------------------------------------------------

@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part needs. ``role`` is ``"matrix"`` (an operand of a
    contraction or an embedding table: held in the compute dtype), ``"vector"``
    (a norm weight or the like: a tensor stored in 32-bit stays 32-bit) or
    ``"table"`` (integers: held as int32). ``init`` describes the random-weights
    mode: ``("normal", std)``, ``("ones",)`` or ``("normal_about_one", std)``."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)


@dataclass(frozen=True)
class PagedKV:
    """A mixer that keeps one key and one value vector per position.
    ``window``: positions a query may look back over, itself included
    (garuda/src/cache/mod.rs:333-338); ``None`` keeps everything."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """A mixer that keeps a state of fixed size per request
    (garuda/src/cache/mod.rs:630-648 is the reference's example)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class LayerCache:
    """What one layer call sees of the cache during a step.

    For ``PagedKV``: ``k`` and ``v`` are this call's slices of its group's page
    pool, ``[num_pages, kv_heads, page_size, head_dim]``; ``block_table`` is the
    group's table for the requests of the batch, ``[R, max_pages]`` int32 (-1
    where a page has been given back). ``writes`` is False for a call that reads
    another call's cache. For ``FixedState``: ``state`` is ``[max_slots, *shape]``
    and the batch's ``slots`` index it.
    """
    need: object
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    block_table: Optional[torch.Tensor] = None
    page_size: int = 0
    state: Optional[torch.Tensor] = None
    writes: bool = True


# --------------------------------------------------------------------------
# base classes
# --------------------------------------------------------------------------

class Part:
    """Common behaviour: tensors by local name, bound once after loading."""

    #: Whether a decode step through this part may be captured in a CUDA graph and replayed: every
    #: launch must read the batch from the device arrays of ``ctx.batch`` only (a replayed step has
    #: no host copies, ``ctx.batch.host`` is empty), launch the same kernels whatever the batch
    #: holds, and allocate nothing. The built-in parts say True; a part that says nothing is run
    #: kernel by kernel.
    graph_safe = False

    def tensors(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], ops, dtype: torch.dtype) -> None:
        """Receive the device tensors named by ``tensors()`` (already in the dtype
        their role asks for). ``ops`` is the kernel set, ``dtype`` the compute dtype."""
        self.ops = ops
        self.dtype = dtype


class Norm(Part):
    def forward(self, ctx, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``x`` is the 32-bit residual stream ``[T, d]``; returns ``[T, d]`` (or
        ``[len(rows), d]``) in the compute dtype."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns positions into a change of the query and key vectors."""
    #: a rotary encoding that the fused rotate-and-store kernel can apply
    rotary = None
    #: False for an encoding that leaves queries and keys alone
    changes_vectors = True

    def apply(self, ctx, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """In place on ``q [T, Hq, hd]`` and ``k [T, Hkv, hd]`` (32-bit)."""
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        """``PagedKV``, ``FixedState`` or ``None``."""
        return None

    def forward(self, ctx, h: torch.Tensor, cache: Optional[LayerCache],
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """``h``: normed input ``[T, d]`` in the compute dtype. Either returns
        the output ``[T, d]`` or, when ``residual`` (32-bit ``[T, d]``) is given
        and the part can add into it itself, adds there and returns ``None``."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, h: torch.Tensor,
                residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        raise NotImplementedError


# --------------------------------------------------------------------------
# registries: name -> class
# --------------------------------------------------------------------------

_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position_encoding": {}, "block": {},
}


def _register(kind: str, name: str, cls=None):
    def deco(c):
        _REGISTRIES[kind][name] = c
        return c
    return deco(cls) if cls is not None else deco


def register_mixer(name, cls=None): return _register("mixer", name, cls)
def register_feed_forward(name, cls=None): return _register("feed_forward", name, cls)
def register_norm(name, cls=None): return _register("norm", name, cls)
def register_position_encoding(name, cls=None): return _register("position_encoding", name, cls)
def register_block(name, cls=None): return _register("block", name, cls)


@dataclass(frozen=True)
class PartSpec:
    """A part named as data: registry ``kind``, registered ``name``, constructor
    parameters, and the prefix its tensor names get in the checkpoint."""
    name: str
    params: dict = field(default_factory=dict)
    prefix: str = ""


def build_part(kind: str, spec: PartSpec):
    try:
        cls = _REGISTRIES[kind][spec.name]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[kind])) or "none"
        raise KeyError(f"no {kind} named '{spec.name}' is registered (registered: {known})") from None
    return cls(**spec.params)
