"""Named ranges on a profiler's timeline (NVTX), switched on with LAYOVER_B200_NVTX=1.

The reference marks its hot path the same way behind LAYOVER_NVTX (layover/profiling.py:14-39).
Here the switch is read once, the first time it is asked for; `active()` lets a hot loop skip
the range altogether, and `nvtx_range(name)` is an ordinary context manager around
`torch.cuda.nvtx.range` that does nothing while the switch is off.
"""

from __future__ import annotations

import os
from contextlib import contextmanager

SWITCH = "LAYOVER_B200_NVTX"
_active: bool | None = None


def active() -> bool:
    """Whether ranges are emitted in this process."""
    global _active
    if _active is None:
        _active = os.environ.get(SWITCH, "") == "1"
    return _active


def set_active(on: bool | None) -> None:
    """Override the environment (None: read it again at the next question)."""
    global _active
    _active = on


@contextmanager
def nvtx_range(name: str):
    if not active():
        yield
        return
    import torch

    with torch.cuda.nvtx.range(name):
        yield
