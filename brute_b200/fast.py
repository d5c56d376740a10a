"""Dispatch-free entry points for hot loops (surface of the reference's ``brute/fast.py``).

These call ``torch.ops.brute.*`` straight on the packed buffers and skip
``__torch_function__``. As in the reference they do not validate: inputs must be
bit1 tensors of matching shape. On CUDA the element-wise ones are single fused
kernels (``eq`` is one XNOR pass, not xor + not).
"""
from __future__ import annotations

import torch

from .tensor import Tensor, _OP_AND, _OP_OR, _OP_XOR, _OP_XNOR, _packed_bin

_ops = torch.ops.brute


# Shapes and packed buffers are read through the plain alias of a tensor (one as_subclass): every
# attribute read on the subclass itself is a __torch_function__ round trip.
def _pk(t: Tensor):
    """(packed buffer, logical shape) of a bit1 tensor."""
    plain = torch.Tensor.as_subclass(t, torch.Tensor)     # the raw one: no materialisation
    return t._packed_fast(plain), plain.shape


def _bin(code: int, a: Tensor, b: Tensor) -> Tensor:
    pa, shape = _pk(a)
    pb, _ = _pk(b)
    return Tensor._make_bit1_from_packed(_packed_bin(code, pa, pb, shape[-1]), shape)


def bitwise_xor(a: Tensor, b: Tensor) -> Tensor:
    """``a ^ b`` on two same-shape bit1 tensors; the result's bool view is lazy."""
    return _bin(_OP_XOR, a, b)


def bitwise_and(a: Tensor, b: Tensor) -> Tensor:
    return _bin(_OP_AND, a, b)


def bitwise_or(a: Tensor, b: Tensor) -> Tensor:
    return _bin(_OP_OR, a, b)


def bitwise_not(a: Tensor) -> Tensor:
    """``~a`` with the pad bits of each row's last word kept 0."""
    pa, shape = _pk(a)
    return Tensor._make_bit1_from_packed(_ops.bit1_not_packed(pa, shape[-1]), shape)


def eq(a: Tensor, b: Tensor) -> Tensor:
    """``a == b``: pad-safe XNOR."""
    return _bin(_OP_XNOR, a, b)


def ne(a: Tensor, b: Tensor) -> Tensor:
    """``a != b``: XOR."""
    return _bin(_OP_XOR, a, b)


def popcount(a: Tensor) -> Tensor:
    """Total number of set bits, 0-dim int64."""
    return Tensor._make_plain(_ops.packed_popcount(_pk(a)[0]))


def hamming(a: Tensor, b: Tensor) -> Tensor:
    """Total Hamming distance, 0-dim int64."""
    return Tensor._make_plain(_ops.bit1_hamming_total(_pk(a)[0], _pk(b)[0]))


def matmul(a: Tensor, b_t: Tensor) -> torch.Tensor:
    """A (M, K) times B given as (N, K) rows of output features -> int32 ``K - 2H``."""
    pa, shape = _pk(a)
    return _ops.xnor_popcount_matmul(pa, _pk(b_t)[0], shape[-1])


def signed_bundle(W: torch.Tensor, V: Tensor) -> Tensor:
    """``out[..., m, :] = sign(sum_n W[..., m, n] * pm1(V[..., n, :]))`` (int8 weights x bit1)."""
    B, M = int(W.shape[0]), int(W.shape[1])
    D = int(V.shape[-1])
    out = _ops.signed_bundle(W.to(torch.int8).contiguous(), V._packed_buf_contig(), D)
    return Tensor._make_bit1_from_packed(out, [B, M, D])


def xor_packed(a_buf: torch.Tensor, b_buf: torch.Tensor) -> torch.Tensor:
    """Raw packed XOR on ``_packed_buf`` tensors, no wrapping."""
    return torch.bitwise_xor(a_buf, b_buf)


def and_packed(a_buf: torch.Tensor, b_buf: torch.Tensor) -> torch.Tensor:
    return torch.bitwise_and(a_buf, b_buf)


def or_packed(a_buf: torch.Tensor, b_buf: torch.Tensor) -> torch.Tensor:
    return torch.bitwise_or(a_buf, b_buf)


def matmul_packed(a_buf: torch.Tensor, b_buf: torch.Tensor, K: int) -> torch.Tensor:
    """Raw packed GEMM, for CUDA-graph captures that hold the packed buffers."""
    return _ops.xnor_popcount_matmul(a_buf, b_buf, K)


__all__ = [
    "bitwise_xor", "bitwise_and", "bitwise_or", "bitwise_not",
    "eq", "ne",
    "popcount", "hamming",
    "matmul",
    "xor_packed", "and_packed", "or_packed", "matmul_packed",
]
