"""Runs the sampling kernels over the logits rows of a step."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


class Sampler:
    def __init__(self, ops, device):
        self.ops, self.device = ops, torch.device(device)
        self._scratch = None

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
               top_p: Sequence[float], u: Sequence[float]) -> List[int]:
        """One token per row of ``logits [R, vocab]`` (float32, on the device).
        Rows with temperature 0 are greedy; ``u`` holds each row's uniform draw."""
        R, V = logits.shape
        if R == 0:
            return []
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        if all(t == 0.0 for t in temperature):
            self.ops.argmax(logits, out)
            return out.tolist()
        host = np.empty((4, R), dtype=np.float32)
        host[0], host[1], host[2] = temperature, top_p, u
        host[3] = np.asarray(top_k, dtype=np.int32).view(np.float32)
        params = torch.from_numpy(host)
        params = params.pin_memory().to(self.device, non_blocking=True) if self.device.type == "cuda" else params
        if self._scratch is None or self._scratch.numel() < R * V:
            self._scratch = torch.empty(R * V, dtype=torch.float32, device=self.device)
        self.ops.sample(logits, params[0], params[3].view(torch.int32), params[1], params[2], out,
                        self._scratch)
        return out.tolist()
