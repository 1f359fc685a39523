"""Choosing the next token of each request from its logits, on the device.

Greedy is the first index of the maximum, as the reference's `argmax` (layover/engine.py:139-141,
187). The reference takes `temperature` in its API and ignores it (layover/server.py:13-14); here
a temperature T > 0 draws from softmax(logits / T) with the Gumbel-max rule and a counter-based
generator keyed by the request's seed and the number of tokens it has sampled so far, so a
request's tokens are the same whatever else is in the batch.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    seed: int = 0


class Sampler:
    def __init__(self, device: torch.device | str):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ops.KernelError("the sampler runs on a CUDA device only")

    def __call__(self, logits: torch.Tensor, params: list[SamplingParams], steps: list[int]) -> list[int]:
        """One token per row of `logits` [R, V]; `steps[r]` is how many tokens row r's request has
        sampled before this one. One copy in, one copy out."""
        return self.launch(logits, params, steps).result()

    def launch(self, logits: torch.Tensor, params: list[SamplingParams], steps: list[int]) -> "PendingTokens":
        """Sample without waiting: the tokens stay on the device (the next step may read them
        there) and travel to pinned host memory behind the kernel; `result()` waits for them."""
        rows = logits.shape[0]
        if rows == 0:
            return PendingTokens(None, None, None)
        if len(params) != rows or len(steps) != rows:
            raise ValueError("one SamplingParams and one step count per row of logits")
        tokens = torch.empty(rows, dtype=torch.int32, device=self.device)
        if all(p.temperature == 0.0 for p in params):
            ops.sample(logits, None, None, None, None, tokens)
        else:
            host = torch.empty((4, rows), dtype=torch.int32, pin_memory=True)
            host[0] = torch.tensor([p.temperature for p in params], dtype=torch.float32).view(torch.int32)
            host[1] = torch.tensor([_signed(p.seed & 0xFFFFFFFF) for p in params], dtype=torch.int32)
            host[2] = torch.tensor([_signed((p.seed >> 32) & 0xFFFFFFFF) for p in params], dtype=torch.int32)
            host[3] = torch.tensor([_signed(s & 0xFFFFFFFF) for s in steps], dtype=torch.int32)
            dev = host.to(self.device, non_blocking=True)
            ops.sample(logits, dev[0].view(torch.float32), dev[1], dev[2], dev[3], tokens)
        host = torch.empty(rows, dtype=torch.int32, pin_memory=True)
        host.copy_(tokens, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return PendingTokens(tokens, host, event)


class PendingTokens:
    """Sampled tokens on their way to the host."""

    def __init__(self, device, host, event):
        self.device, self._host, self._event = device, host, event

    def result(self) -> list[int]:
        if self._host is None:
            return []
        self._event.synchronize()
        return self._host.tolist()


def _signed(word: int) -> int:
    return word - (1 << 32) if word >= (1 << 31) else word
