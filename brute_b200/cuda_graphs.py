"""CUDA-graph helpers (surface of the reference's ``brute/cuda_graphs.py``).

``capture(fn, warmup)`` runs ``fn`` a few times, records one more run into a
``torch.cuda.CUDAGraph`` on a side stream and returns the graph with the
recorded outputs on ``.outputs``; ``replay(g)`` relaunches it. The launchers of
this package never synchronise or allocate outside torch's caching allocator,
so they can be captured.
"""
from __future__ import annotations

from typing import Any, Callable

import torch


def capture(fn: Callable[[], Any], warmup: int = 3) -> "torch.cuda.CUDAGraph":
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA Graphs require a CUDA build of PyTorch")
    for _ in range(max(0, int(warmup))):
        fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph):
            outputs = fn()
    torch.cuda.current_stream().wait_stream(side)
    graph.outputs = outputs          # type: ignore[attr-defined]
    return graph


def replay(g: "torch.cuda.CUDAGraph") -> Any:
    g.replay()
    return getattr(g, "outputs", None)


__all__ = ["capture", "replay"]
