"""Round-robin CUDA streams for independent bit1 op chains.

Surface of the reference's ``brute/streams.py``: ``parallel_streams(n, device)``
is a context manager that makes every lookup of the current stream return the
next stream of a cached pool, so consecutive independent ops land on different
streams; on exit the caller's stream waits for all of them. Without CUDA it is a
no-op.

The reference patches the same function, but its compiled ops ask the runtime for the current
stream, so there the rotation never reaches a kernel. Here it does: while a block is active every
``torch.ops.brute.*`` call (Python binding) takes the next pool stream and runs ENTIRELY on it --
the pool stream is made the real current stream for the duration of the call, so the caching
allocator, any ATen helper inside the op and the kernel launch agree on the stream. Ordering is kept
by events, never by luck:

* before the call the pool stream waits for everything queued so far on the caller's stream (ATen
  work inside the block) and for the producer of every input that an earlier call of the block made
  on another pool stream (a dependent chain such as ``(x & y) ^ z``);
* every input is marked as used on the pool stream (``record_stream``), so that freeing it inside
  the block cannot hand its memory to a kernel that runs before this one has finished;
* ``join()`` makes the caller's stream wait for all pool work queued so far; the front end calls it
  before it hands bit1 data to a plain torch op inside the block, and the block calls it on exit.
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


_REAL_CURRENT_STREAM = torch.cuda.current_stream      # the unpatched function
_ACTIVE: Optional["_Rotator"] = None                  # the innermost active block, if any


def _storage_ptr(t: torch.Tensor) -> int:
    """Address of the first byte of the tensor's storage (views of one allocation share it)."""
    return t.data_ptr() - t.storage_offset() * t.element_size()


class _Rotator:
    """Hands out the pool's streams in turn and keeps the block's ordering state."""

    def __init__(self, streams, device):
        self.streams = streams
        self.device = device
        self._cycle = itertools.cycle(range(len(streams)))
        self.idx = 0
        self._producers: Dict[int, Tuple["torch.cuda.Stream", "torch.cuda.Event"]] = {}
        self._tail: Dict[int, "torch.cuda.Event"] = {}

    def next(self) -> "torch.cuda.Stream":
        self.idx = next(self._cycle)
        return self.streams[self.idx]

    # -- called by the op layer -------------------------------------------------------------------
    def run(self, fn, args):
        """Run one op (allocation + launch) on the next pool stream, ordered after its inputs."""
        tensors = [a for a in args if isinstance(a, torch.Tensor) and a.is_cuda]
        if not tensors or tensors[0].device != self.device:
            return fn(*args)
        s = self.next()
        outer = _REAL_CURRENT_STREAM(self.device)
        if outer.cuda_stream != s.cuda_stream:
            s.wait_event(outer.record_event())
        for t in tensors:
            prod = self._producers.get(_storage_ptr(t))
            if prod is not None and prod[0] is not s:
                s.wait_event(prod[1])
            t.record_stream(s)
        torch.cuda.set_stream(s)
        try:
            out = fn(*args)
        finally:
            torch.cuda.set_stream(outer)
        done = s.record_event()
        self._tail[id(s)] = done
        for o in (out if isinstance(out, (tuple, list)) else (out,)):
            if isinstance(o, torch.Tensor) and o.is_cuda:
                self._producers[_storage_ptr(o)] = (s, done)
        if len(self._producers) > 4096:            # bounded: older producers are covered by join()
            self.join()
        return out

    def join(self) -> None:
        """The caller's stream waits for all pool work queued so far."""
        outer = _REAL_CURRENT_STREAM(self.device)
        for ev in self._tail.values():
            outer.wait_event(ev)
        self._tail.clear()
        self._producers.clear()


def active() -> Optional[_Rotator]:
    """The rotator of the innermost ``parallel_streams`` block, or None."""
    return _ACTIVE


def join_active() -> None:
    """Order the caller's stream after the active block's pool work (no-op outside a block)."""
    if _ACTIVE is not None:
        _ACTIVE.join()


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
    global _ACTIVE
    rot = _Rotator(pool, device)
    original = torch.cuda.current_stream
    previous = _ACTIVE

    def rotating(device=None):
        return rot.next()

    torch.cuda.current_stream = rotating            # type: ignore[assignment]
    _ACTIVE = rot
    try:
        yield rot
    finally:
        _ACTIVE = previous
        torch.cuda.current_stream = original        # type: ignore[assignment]
        for s in pool:
            outer.wait_stream(s)


__all__ = ["parallel_streams"]
