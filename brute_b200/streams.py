"""Round-robin CUDA streams for independent bit1 op chains.

Surface of the reference's ``brute/streams.py``: ``parallel_streams(n, device)``
is a context manager that makes every lookup of the current stream return the
next stream of a cached pool, so consecutive independent ops land on different
streams; on exit the caller's stream waits for all of them. Without CUDA it is a
no-op. Every kernel of this package launches on ``torch.cuda.current_stream``,
so it rotates with the pool.
"""
from __future__ import annotations

import contextlib
import itertools
from typing import Dict, List, Optional, Tuple

import torch

_POOLS: Dict[Tuple[int, int], List["torch.cuda.Stream"]] = {}


def _get_pool(device: torch.device, n: int) -> List["torch.cuda.Stream"]:
    if device.type != "cuda":
        raise RuntimeError("parallel_streams only supported on CUDA")
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, n)
    if key not in _POOLS:
        _POOLS[key] = [torch.cuda.Stream(device=device) for _ in range(n)]
    return _POOLS[key]


class _Rotator:
    """Hands out the pool's streams in turn."""

    def __init__(self, streams):
        self.streams = streams
        self._cycle = itertools.cycle(range(len(streams)))
        self.idx = 0

    def next(self) -> "torch.cuda.Stream":
        self.idx = next(self._cycle)
        return self.streams[self.idx]


@contextlib.contextmanager
def parallel_streams(n: int = 4, device: Optional[torch.device] = None):
    if not torch.cuda.is_available():
        yield
        return
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    pool = _get_pool(device, max(1, int(n)))
    outer = torch.cuda.current_stream(device=device)
    for s in pool:                       # work queued before the block is visible to the pool
        s.wait_stream(outer)
    rot = _Rotator(pool)
    original = torch.cuda.current_stream

    def rotating(device=None):
        return rot.next()

    torch.cuda.current_stream = rotating            # type: ignore[assignment]
    try:
        yield rot
    finally:
        torch.cuda.current_stream = original        # type: ignore[assignment]
        for s in pool:
            outer.wait_stream(s)


__all__ = ["parallel_streams"]
