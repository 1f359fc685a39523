"""NVTX ranges for a profiler's timeline, off unless LAYOVER_B200_NVTX=1 (the reference gates its
ranges the same way with LAYOVER_NVTX, layover/profiling.py:14-39). Off, a range is one shared
do-nothing context manager."""

from __future__ import annotations

import os
from contextlib import nullcontext

ENABLED = os.environ.get("LAYOVER_B200_NVTX") == "1"
_OFF = nullcontext()


class _Range:
    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


def nvtx_range(name: str):
    return _Range(name) if ENABLED else _OFF
