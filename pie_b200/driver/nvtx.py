"""NVTX ranges around the driver's phases, for timelines taken with an external profiler. Off unless
`PIE_NVTX=1`: a disabled range is one attribute test. The ranges: `pie.fire` > {`build`, `forward.decode` |
`forward.general`, `respond`}, `pie.decode.launch` (a pipelined decode step) and `pie.copy`.
Counterpart of the NVTX build option of the reference's CUDA driver (driver/cuda/CMakeLists.txt, PIE_NVTX).
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Callable, Optional, Tuple

_push: Optional[Callable[[str], object]] = None
_pop: Optional[Callable[[], object]] = None


def enable(backend: Optional[Tuple[Callable[[str], object], Callable[[], object]]] = None) -> bool:
    """Turn ranges on: through `torch.cuda.nvtx` when a GPU is present, or through a given (push, pop) pair."""
    global _push, _pop
    if backend is not None:
        _push, _pop = backend
        return True
    import torch
    if torch.cuda.is_available():
        _push, _pop = torch.cuda.nvtx.range_push, torch.cuda.nvtx.range_pop
        return True
    return False


def disable() -> None:
    global _push, _pop
    _push = _pop = None


@contextmanager
def range(name: str):
    if _push is None:
        yield
        return
    _push(name)
    try:
        yield
    finally:
        _pop()


if os.environ.get("PIE_NVTX") == "1":
    enable()
