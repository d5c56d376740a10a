"""Second, independent restatement of the path in plain numpy (small sizes).

TEST INFRASTRUCTURE ONLY. It exists to cross-check ``c_oracle`` and to state the
semantics in the most literal way: unpack everything to one bool per bit and use
integer arithmetic. Reference lines are cited per function.
"""
from __future__ import annotations

import numpy as np


def pack_bool(x: np.ndarray) -> np.ndarray:
    """LSB-first, 64 bits per word along the last axis, zero pad bits
    (cbrute/cpu/kernels/packing.hpp:3-6, cbrute/cpu/ops_cpu.cpp:39-70)."""
    x = np.asarray(x) != 0
    ld = x.shape[-1]
    wpr = (ld + 63) // 64
    pad = wpr * 64 - ld
    xb = np.concatenate([x, np.zeros(x.shape[:-1] + (pad,), dtype=bool)], axis=-1)
    by = np.packbits(xb, axis=-1, bitorder="little")
    return np.ascontiguousarray(by).view(np.uint64).reshape(x.shape[:-1] + (wpr,))


def unpack_bool(p: np.ndarray, shape) -> np.ndarray:
    """cbrute/cpu/kernels/packing.hpp:159-171"""
    p = np.ascontiguousarray(p).view(np.uint64)
    ll = int(shape[-1])
    bits = np.unpackbits(p.view(np.uint8).reshape(p.shape[:-1] + (-1,)), axis=-1, bitorder="little")
    return bits[..., :ll].astype(bool).reshape(shape)


def unpack_pm1(p: np.ndarray, shape) -> np.ndarray:
    """+1.0 for a set bit, -1.0 otherwise (cbrute/cpu/kernels/packing.hpp:139-156)."""
    return np.where(unpack_bool(p, shape), np.float32(1), np.float32(-1))


def sign_bits(x: np.ndarray, mode: int) -> np.ndarray:
    """mode 0: x > 0 (brute/tensor.py:163-169); mode 1: x >= 0 (brute/functional.py:131-133)."""
    return (x >= 0) if mode else (x > 0)


def popcount_words(x: np.ndarray) -> np.ndarray:
    """Per-element popcount on the unsigned bit pattern (cbrute/cuda/kernels/popcount.cuh:22-41)."""
    x = np.ascontiguousarray(x)
    u8 = x.view(np.uint8).reshape(x.shape + (x.dtype.itemsize,))
    return np.unpackbits(u8, axis=-1).sum(axis=-1).astype(np.int32)


def xnor_gemm(a_bool: np.ndarray, b_bool: np.ndarray) -> np.ndarray:
    """The +-1 dot product, K - 2*H (cbrute/cuda/kernels/matmul_fallback.cuh:5-6),
    from unpacked bools: A [M,K], B [N,K] -> int32 [M,N]."""
    a = np.where(a_bool, 1, -1).astype(np.int32)
    b = np.where(b_bool, 1, -1).astype(np.int32)
    return (a @ b.T).astype(np.int32)


def not_masked(p: np.ndarray, last_dim_bits: int) -> np.ndarray:
    """cbrute/ext.cpp:27-39"""
    out = ~np.ascontiguousarray(p).view(np.uint64)
    vb = last_dim_bits % 64
    if out.size and last_dim_bits and vb:
        out[..., -1] &= np.uint64((1 << vb) - 1)
    return out


def binary_attention(q_bool, k_bool, V, causal: bool, scale: float) -> np.ndarray:
    """Composition oracle (no reference kernel exists): +-1 scores * scale, causal
    mask, fp32 softmax, @ V. q_bool, k_bool [B,H,S,D] bool; V float32."""
    q = np.where(q_bool, 1.0, -1.0).astype(np.float32)
    k = np.where(k_bool, 1.0, -1.0).astype(np.float32)
    s = np.einsum("bhid,bhjd->bhij", q, k) * np.float32(scale)
    if causal:
        S = s.shape[-1]
        s = np.where(np.tril(np.ones((S, S), dtype=bool)), s, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    p = p / p.sum(axis=-1, keepdims=True)
    return np.einsum("bhij,bhjd->bhid", p, V.astype(np.float32)).astype(np.float32)
