"""Random-weights mode: write a model folder from a configuration and a seed.

The reference's synthetic mode draws weights from a seeded splitmix64
(garuda/src/weights/mod.rs:17-40, :70-83). Here every tensor has a generator of
its own, keyed by the seed and the tensor's name, so that the values of a
tensor depend on neither the order of the tensors nor on which others exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Optional

import numpy as np
import torch

from ..config.registry import build_model
from .safetensors_io import write_safetensors


def _generator(seed: int, name: str) -> np.random.Generator:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return np.random.Generator(np.random.Philox(key=int.from_bytes(digest[:16], "little")))


def random_tensor(seed: int, name: str, shape, init) -> torch.Tensor:
    kind = init[0]
    rng = _generator(seed, name)
    if kind == "ones":
        a = np.ones(shape, dtype=np.float32)
    elif kind == "normal":
        a = rng.standard_normal(shape, dtype=np.float32) * np.float32(init[1])
    elif kind == "normal_about_one":
        a = np.float32(1.0) + rng.standard_normal(shape, dtype=np.float32) * np.float32(init[1])
    else:
        raise ValueError(f"unknown initialiser {init!r}")
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))


def random_weights(config_dict: dict, seed: int, norm_init=None, store_dtype=torch.float32,
                   scale: Optional[Dict[str, float]] = None) -> Dict[str, torch.Tensor]:
    """CPU tensors for every name the model expects. ``norm_init`` overrides the
    initialiser of vectors (norm weights), e.g. ``("normal_about_one", 0.1)``.
    ``scale``: factors for the tensors whose name contains a key, e.g.
    ``{"q_proj": 8.0, "k_proj": 8.0}``: with N(0, 0.02) weights the attention
    scores of a small model are so close to zero that every key weighs the same,
    and a fault in positions, rotation or masking barely moves the logits."""
    _, model = build_model(config_dict)
    out = {}
    for name, ts in model.expected_tensors().items():
        init = tuple(norm_init) if (norm_init is not None and ts.role == "vector") else ts.init
        t = random_tensor(seed, name, ts.shape, init)
        for key, factor in (scale or {}).items():
            if key in name:
                t = t * float(factor)
        out[name] = t.to(store_dtype)
    return out


def write_random_model(model_dir: str, config_dict: dict, seed: int, norm_init=None,
                       store_dtype=torch.float32, scale: Optional[Dict[str, float]] = None) -> str:
    """Create ``model_dir`` with config.json and model.safetensors."""
    os.makedirs(model_dir, exist_ok=True)
    tensors = random_weights(config_dict, seed, norm_init, store_dtype, scale)
    with open(os.path.join(model_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=2)
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return model_dir
