"""Packed on-disk form of bit1 tensors.

Pickling a bit1 tensor the reference's way stores its bool storage (``__reduce_ex__``,
brute/tensor.py:2073-2081): one byte per bit. ``save_packed`` writes the packed words instead,
64 bits per int64, so a binarised weight file is 8x smaller and loading it never touches a
bool: the tensor is rebuilt around the packed buffer and unpacks only if someone reads it as bool.

The file is an ordinary ``torch.save`` of plain containers, tensors and primitives (loadable with
``weights_only=True``); a bit1 tensor is the dict ``{"__bit1__": 1, "shape": [...], "packed": int64}``.
"""
from __future__ import annotations

from typing import Any

import torch

from .tensor import Tensor, _is_b1

_TAG = "__bit1__"


def _encode(obj: Any) -> Any:
    if isinstance(obj, Tensor) and _is_b1(obj):
        packed = obj._packed_buf_contig()
        return {_TAG: 1, "shape": [int(s) for s in obj.shape], "packed": packed.detach().cpu()}
    if isinstance(obj, torch.Tensor):
        return obj.as_subclass(torch.Tensor).detach().cpu()
    if isinstance(obj, dict):
        if _TAG in obj:
            raise ValueError(f"save_packed: the key {_TAG!r} is reserved")
        return {k: _encode(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_encode(v) for v in obj)
    return obj


def _decode(obj: Any, device) -> Any:
    if isinstance(obj, dict):
        if obj.get(_TAG) == 1:
            packed = obj["packed"]
            shape = [int(s) for s in obj["shape"]]
            words = (shape[-1] + 63) // 64 if shape else 1
            if packed.dtype != torch.int64 or list(packed.shape) != (shape[:-1] + [words] if shape else [1]):
                raise ValueError("load_packed: packed buffer does not match the logical shape")
            if device is not None:
                packed = packed.to(device)
            return Tensor._make_bit1_from_packed(packed, shape)
        return {k: _decode(v, device) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_decode(v, device) for v in obj)
    if isinstance(obj, torch.Tensor):
        t = obj.to(device) if device is not None else obj
        return Tensor._make_plain(t)
    return obj


def save_packed(obj: Any, f) -> None:
    """Save a bit1 tensor, or any nesting of dicts / lists / tuples of tensors, in packed form."""
    torch.save(_encode(obj), f)


def load_packed(f, device=None) -> Any:
    """Load what ``save_packed`` wrote; bit1 tensors come back packed-only on ``device``.

    With the default (``device=None``) the packed words stay in host memory. The package has CUDA
    kernels only, so such a tensor can be moved (``t.to("cuda")`` carries the packed words, an eighth
    of the bool bytes, and leaves the bool view lazy) but not computed with or read as bool before it
    has been moved: pass ``device="cuda"`` to load straight onto the GPU."""
    return _decode(torch.load(f, map_location="cpu", weights_only=True), device)
