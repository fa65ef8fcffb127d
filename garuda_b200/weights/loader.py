"""Weights from a model folder, by tensor name.

The reference looks every tensor up by name and checks its element count
(garuda/src/llama/mod.rs:358-381, :298-310), stopping at the first problem.
Here all problems of a folder are collected and reported in one error: tensors
that are missing, tensors nobody asked for, and tensors of the wrong shape.

Dtypes: a matrix (operand of a matrix product, or the embedding table) is held
in the compute dtype, bfloat16 or float32. A vector (norm weight) that the file
stores in 32-bit stays 32-bit, otherwise it takes the compute dtype. Integer
tables are held as int32.
"""
from __future__ import annotations

import os
from typing import Dict

import torch

from ..config.model_config import read_config_json
from ..config.registry import build_model
from .safetensors_io import SafetensorsFolder, SafetensorsError


class WeightError(ValueError):
    """Lists every missing, unexpected and wrongly shaped tensor of a folder."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"weights in {model_dir} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in self.wrong_shape))
        for o in other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


_FLOATS = (torch.float32, torch.float16, torch.bfloat16, torch.float64)


def target_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if role == "table":
        return torch.int32
    if role == "vector" and stored == torch.float32:
        return torch.float32
    return compute


def check_folder(model, folder: SafetensorsFolder, tied_ok: bool = True):
    """Compare the folder's tensors with what the model expects."""
    expected = model.expected_tensors()
    have = folder.entries
    missing = [n for n in expected if n not in have]
    # what the architecture says a folder may carry unread (a tied model's copy of its head, which
    # is the embedding table) is not unexpected
    ignored = set(getattr(model.spec, "ignored_tensors", ())) if tied_ok else set()
    unexpected = [n for n in have if n not in expected and n not in ignored]
    wrong, other = [], []
    for n, ts in expected.items():
        if n in have:
            e = have[n]
            if tuple(e.shape) != tuple(ts.shape):
                wrong.append((n, e.shape, ts.shape))
            elif ts.role != "table" and e.torch_dtype not in _FLOATS:
                other.append(f"{n}: stored as {e.dtype}, which is not a floating-point type")
    return missing, unexpected, wrong, other


def load_weights(model, model_dir: str, ops, dtype: torch.dtype, device) -> None:
    """Read every tensor the model names, move it to the device in the dtype its
    role asks for, and hand it to the parts."""
    try:
        folder = SafetensorsFolder(model_dir)
    except SafetensorsError as e:
        raise WeightError(model_dir, [], [], [], other=[str(e)]) from None
    missing, unexpected, wrong, other = check_folder(model, folder)
    if missing or unexpected or wrong or other:
        raise WeightError(model_dir, missing, unexpected, wrong, other)
    tensors: Dict[str, torch.Tensor] = {}
    for name, ts in model.expected_tensors().items():
        cpu = folder.tensor(name)
        want = target_dtype(ts.role, cpu.dtype, dtype)
        t = cpu.to(device=device, dtype=want, copy=True).contiguous()
        if ts.role != "table" and not bool(torch.isfinite(t).all()):
            raise WeightError(model_dir, [], [], [], other=[f"{name}: holds values that are not finite"])
        tensors[name] = t
    model.load(tensors, ops, dtype)


def load_model(model_dir: str, ops, dtype: torch.dtype, device):
    """(typed configuration, Decoder with weights) from a folder with
    config.json and model.safetensors; the class is chosen by config.json."""
    cfg, model = build_model(read_config_json(model_dir))
    load_weights(model, model_dir, ops, dtype, device)
    return cfg, model
