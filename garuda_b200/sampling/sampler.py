"""Runs the sampling kernels over the logits rows of a step."""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch


class Pending:
    """Tokens on their way: on the device at once (``tokens``), on the host once
    ``done`` has passed."""

    def __init__(self, tokens, host, done):
        self.tokens, self.host, self.done = tokens, host, done


class Sampler:
    def __init__(self, ops, device):
        self.ops, self.device = ops, torch.device(device)
        self._scratch = None
        self._staging = {}       # pinned buffers for the tokens' way back, two per size in turn
        self._turn = 0
        self._params, self._params_turn = {}, 0      # pinned buffers for the rows' sampling parameters

    def _host_buffer(self, R: int) -> torch.Tensor:
        self._turn ^= 1
        key = (R, self._turn)
        if key not in self._staging:
            self._staging[key] = torch.empty(R, dtype=torch.int32).pin_memory()
        return self._staging[key]

    def launch(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
               top_p: Sequence[float], u: Sequence[float]) -> Pending:
        """Starts drawing one token per row of ``logits [R, vocab]`` and their copy to
        the host, and returns without waiting; ``result`` waits. A buffer of its own
        holds the tokens on the device, so that a next step can read them there."""
        R = logits.shape[0]
        out = torch.empty(max(R, 1), dtype=torch.int32, device=self.device)[:R]
        if R == 0:
            return Pending(out, None, None)
        self._draw(logits, temperature, top_k, top_p, u, out)
        if self.device.type != "cuda":
            return Pending(out, out, None)
        host = self._host_buffer(R)
        host.copy_(out, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return Pending(out, host, done)

    @staticmethod
    def result(pending: Pending) -> List[int]:
        if pending.host is None:
            return []
        if pending.done is not None:
            pending.done.synchronize()
        return pending.host.tolist()

    def sample(self, logits: torch.Tensor, temperature: Sequence[float], top_k: Sequence[int],
               top_p: Sequence[float], u: Sequence[float]) -> List[int]:
        """One token per row of ``logits [R, vocab]`` (float32, on the device).
        Rows with temperature 0 are greedy; ``u`` holds each row's uniform draw."""
        return self.result(self.launch(logits, temperature, top_k, top_p, u))

    def _draw(self, logits, temperature, top_k, top_p, u, out) -> None:
        R, V = logits.shape
        if all(t == 0.0 for t in temperature):
            self.ops.argmax(logits, out)
            return
        if self.device.type == "cuda":
            # pinned buffers kept and taken in turn (pinning memory anew costs more than the kernel); the
            # event tells when the copy that last read a buffer has run
            self._params_turn = (self._params_turn + 1) % 4
            key = (R, self._params_turn)
            slot = self._params.get(key)
            if slot is None:
                slot = self._params[key] = [torch.empty((4, R), dtype=torch.float32).pin_memory(), None]
            if slot[1] is not None:
                slot[1].synchronize()
            pinned = slot[0]
            host = pinned.numpy()
        else:
            host = np.empty((4, R), dtype=np.float32)
        host[0], host[1], host[2] = temperature, top_p, u
        host[3] = np.asarray(top_k, dtype=np.int32).view(np.float32)
        if self.device.type == "cuda":
            params = pinned.to(self.device, non_blocking=True)
            if slot[1] is None:
                slot[1] = torch.cuda.Event()
            slot[1].record()
        else:
            params = torch.from_numpy(host)
        if self._scratch is None or self._scratch.numel() < R * V:
            self._scratch = torch.empty(R * V, dtype=torch.float32, device=self.device)
        small = all(t == 0.0 or 0 < k <= getattr(self.ops, "SMALL_TOP_K", 0) for t, k in zip(temperature, top_k))
        if small:
            self.ops.sample(logits, params[0], params[3].view(torch.int32), params[1], params[2], out,
                            self._scratch, small_top_k=True)
        else:
            self.ops.sample(logits, params[0], params[3].view(torch.int32), params[1], params[2], out,
                            self._scratch)
