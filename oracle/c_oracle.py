"""ctypes wrapper around ``liboracle.so`` (the C restatement of the reference CPU
path). TEST INFRASTRUCTURE ONLY: never imported by the ``brute_b200`` package.

Every function takes and returns numpy arrays; packed buffers are ``uint64``
(or ``int64``, reinterpreted) with 64 bits per word along the last axis.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``brute_oracle.c`` with gcc through the Makefile beside it."""
    src = _DIR / "brute_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B", "liboracle.so"], check=True,
                       capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        L = C.CDLL(str(_LIB_PATH))
        i64, p, i32, f32 = C.c_int64, C.c_void_p, C.c_int, C.c_float
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.argtypes = [i32]
        L.oracle_has_vpopcntdq.restype = C.c_int
        L.oracle_pack_bool.argtypes = [p, p, i64, i64]
        L.oracle_pack_sign_f32.argtypes = [p, p, i64, i64, i32]
        L.oracle_unpack_bool.argtypes = [p, p, i64, i64]
        L.oracle_unpack_pm1_f32.argtypes = [p, p, i64, i64]
        L.oracle_popcount_elems.argtypes = [p, p, i64, i32]
        L.oracle_popcount_total.argtypes = [p, i64]
        L.oracle_popcount_total.restype = C.c_uint64
        L.oracle_hamming_total.argtypes = [p, p, i64]
        L.oracle_hamming_total.restype = C.c_uint64
        L.oracle_hamming_words.argtypes = [p, p, p, i64]
        L.oracle_bitwise.argtypes = [i32, p, p, p, i64, i64, i64]
        L.oracle_select.argtypes = [p, p, p, p, i64]
        L.oracle_row_any.argtypes = [p, p, i64, i64]
        L.oracle_row_all.argtypes = [p, p, i64, i64, i64]
        L.oracle_xnor_gemm.argtypes = [p, p, p, i64, i64, i64, i64, i64]
        L.oracle_xnor_gemm_scale_sign_pack.argtypes = [p, p, p, p, i64, i64, i64, i64, i32]
        L.oracle_signed_bundle.argtypes = [p, p, p, i64, i64, i64, i64, i64]
        L.oracle_binary_attention.argtypes = [p, p, p, p, i64, i64, i64, i32, f32]
        L.oracle_transpose_bits.argtypes = [p, p, i64, i64, i64]
        L.oracle_reduce_rows.argtypes = [i32, p, p, i64, i64, i64]
        L.oracle_move_bits.argtypes = [i32, p, p, p, i64, i64, i64, i64]
        L.oracle_scatter_bits.argtypes = [p, p, p, i32, i64, i64, i64]
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype=None) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a if dtype is None else a.astype(dtype, copy=False)


def _u64(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint64) if a.dtype == np.int64 else a.astype(np.uint64, copy=False)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def has_vpopcntdq() -> bool:
    return bool(lib().oracle_has_vpopcntdq())


def _rows(shape):
    ld = int(shape[-1])
    rows = int(np.prod(shape[:-1], dtype=np.int64)) if len(shape) > 1 else 1
    return rows, ld


def pack_bool(x: np.ndarray) -> np.ndarray:
    """bool/uint8 [..., ld] -> uint64 [..., ceil(ld/64)]."""
    x = _c(x).view(np.uint8) if x.dtype == np.bool_ else _c(x, np.uint8)
    rows, ld = _rows(x.shape)
    wpr = (ld + 63) // 64
    out = np.zeros(x.shape[:-1] + (wpr,), dtype=np.uint64)
    if rows and ld:
        lib().oracle_pack_bool(_ptr(x), _ptr(out), rows, ld)
    return out


def pack_sign_f32(x: np.ndarray, mode: int) -> np.ndarray:
    """float32 [..., ld] -> packed; mode 0: x > 0, mode 1: x >= 0."""
    x = _c(x, np.float32)
    rows, ld = _rows(x.shape)
    wpr = (ld + 63) // 64
    out = np.zeros(x.shape[:-1] + (wpr,), dtype=np.uint64)
    if rows and ld:
        lib().oracle_pack_sign_f32(_ptr(x), _ptr(out), rows, ld, int(mode))
    return out


def unpack_bool(packed: np.ndarray, shape) -> np.ndarray:
    p = _u64(packed)
    shape = tuple(int(s) for s in shape)
    rows, ll = _rows(shape)
    out = np.zeros(shape, dtype=np.uint8)
    if rows and ll:
        lib().oracle_unpack_bool(_ptr(p), _ptr(out), rows, ll)
    return out.view(np.bool_)


def unpack_pm1(packed: np.ndarray, shape) -> np.ndarray:
    p = _u64(packed)
    shape = tuple(int(s) for s in shape)
    rows, ll = _rows(shape)
    out = np.zeros(shape, dtype=np.float32)
    if rows and ll:
        lib().oracle_unpack_pm1_f32(_ptr(p), _ptr(out), rows, ll)
    return out


def popcount_elems(x: np.ndarray) -> np.ndarray:
    x = _c(x)
    if x.dtype == np.bool_:
        x = x.view(np.uint8)
    out = np.zeros(x.shape, dtype=np.int32)
    if x.size:
        lib().oracle_popcount_elems(_ptr(x), _ptr(out), x.size, x.dtype.itemsize)
    return out


def popcount_total(x: np.ndarray) -> int:
    x = _c(x)
    return int(lib().oracle_popcount_total(_ptr(x), x.nbytes)) if x.size else 0


def hamming_total(a: np.ndarray, b: np.ndarray) -> int:
    a, b = _c(a), _c(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    return int(lib().oracle_hamming_total(_ptr(a), _ptr(b), a.nbytes)) if a.size else 0


def hamming_words(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _u64(a), _u64(b)
    out = np.zeros(a.shape, dtype=np.int32)
    if a.size:
        lib().oracle_hamming_words(_ptr(a), _ptr(b), _ptr(out), a.size)
    return out


OPS = {"and": 0, "or": 1, "xor": 2, "xnor": 3, "andnot": 4, "not": 5}


def bitwise(op: str, a: np.ndarray, b, last_dim_bits: int) -> np.ndarray:
    a = _u64(a)
    b = a if b is None else _u64(b)
    out = np.zeros(a.shape, dtype=np.uint64)
    if a.size:
        wpr = a.shape[-1]
        lib().oracle_bitwise(OPS[op], _ptr(a), _ptr(b), _ptr(out), a.size // wpr, wpr, int(last_dim_bits))
    return out


def select(c, a, b) -> np.ndarray:
    c, a, b = _u64(c), _u64(a), _u64(b)
    out = np.zeros(a.shape, dtype=np.uint64)
    if a.size:
        lib().oracle_select(_ptr(c), _ptr(a), _ptr(b), _ptr(out), a.size)
    return out


def row_any(a) -> np.ndarray:
    a = _u64(a)
    wpr = a.shape[-1]
    rows = a.size // wpr if wpr else int(np.prod(a.shape[:-1]))
    out = np.zeros(a.shape[:-1], dtype=np.uint8)
    if rows:
        lib().oracle_row_any(_ptr(a), _ptr(out), rows, wpr)
    return out.view(np.bool_)


def row_all(a, last_dim_bits: int) -> np.ndarray:
    a = _u64(a)
    wpr = a.shape[-1]
    rows = a.size // wpr if wpr else int(np.prod(a.shape[:-1]))
    out = np.zeros(a.shape[:-1], dtype=np.uint8)
    if rows:
        lib().oracle_row_all(_ptr(a), _ptr(out), rows, wpr, int(last_dim_bits))
    return out.view(np.bool_)


def xnor_gemm(A: np.ndarray, B: np.ndarray, K: int) -> np.ndarray:
    """A [M, Kp], B [N, Kp] packed -> int32 [M, N] = K - 2*popcount(a ^ b)."""
    A, B = _u64(A), _u64(B)
    M, Kp = A.shape
    N = B.shape[0]
    assert B.shape[1] == Kp
    out = np.zeros((M, N), dtype=np.int32)
    if M and N:
        lib().oracle_xnor_gemm(_ptr(A), _ptr(B), _ptr(out), M, N, Kp, int(K), N)
    return out


def xnor_gemm_scale_sign_pack(A, B, scale, K: int, mode: int) -> np.ndarray:
    A, B = _u64(A), _u64(B)
    scale = _c(scale, np.float32)
    M, Kp = A.shape
    N = B.shape[0]
    out = np.zeros((M, (N + 63) // 64), dtype=np.uint64)
    if M and N:
        lib().oracle_xnor_gemm_scale_sign_pack(_ptr(A), _ptr(B), _ptr(scale), _ptr(out), M, N, Kp, int(K), int(mode))
    return out


def signed_bundle(W: np.ndarray, V: np.ndarray, D: int) -> np.ndarray:
    """W int8 [B, M, N], V packed [B, N, Dp] -> packed votes [B, M, Dp]."""
    W = _c(W, np.int8)
    V = _u64(V)
    B, M, N = W.shape
    Dp = V.shape[2]
    out = np.zeros((B, M, Dp), dtype=np.uint64)
    if out.size:
        lib().oracle_signed_bundle(_ptr(W), _ptr(V), _ptr(out), B, M, N, Dp, int(D))
    return out


def binary_attention(Qp, Kp, V, causal: bool, scale: float) -> np.ndarray:
    """Qp, Kp [B, H, S, D/64] packed; V float32 [B, H, S, D] -> float32 [B, H, S, D]."""
    Qp, Kp = _u64(Qp), _u64(Kp)
    V = _c(V, np.float32)
    B, H, S, D = V.shape
    out = np.zeros_like(V)
    if out.size:
        lib().oracle_binary_attention(_ptr(Qp), _ptr(Kp), _ptr(V), _ptr(out), B * H, S, D, int(bool(causal)), float(scale))
    return out


def transpose_bits(packed: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """packed [..., rows, ceil(cols/64)] -> packed [..., cols, ceil(rows/64)]."""
    p = _u64(packed)
    batch = int(np.prod(p.shape[:-2], dtype=np.int64)) if p.ndim > 2 else 1
    out = np.zeros(p.shape[:-2] + (int(cols), (int(rows) + 63) // 64), dtype=np.uint64)
    if out.size:
        lib().oracle_transpose_bits(_ptr(p), _ptr(out), batch, int(rows), int(cols))
    return out


def reduce_rows(packed: np.ndarray, dim: int, use_or: bool) -> np.ndarray:
    """OR / AND of packed words over a non-packed axis."""
    p = _u64(packed)
    d = dim % p.ndim
    outer = int(np.prod(p.shape[:d], dtype=np.int64))
    inner = int(np.prod(p.shape[d + 1:], dtype=np.int64))
    out = np.zeros(p.shape[:d] + p.shape[d + 1:], dtype=np.uint64)
    if out.size:
        lib().oracle_reduce_rows(1 if use_or else 0, _ptr(p), _ptr(out), outer, int(p.shape[d]), inner)
    return out


def _move_bits(mode: int, packed: np.ndarray, n_in: int, n_out: int, idx=None, shift: int = 0) -> np.ndarray:
    p = _u64(packed)
    rows = int(np.prod(p.shape[:-1], dtype=np.int64)) if p.ndim > 1 else 1
    out = np.zeros(p.shape[:-1] + ((int(n_out) + 63) // 64,), dtype=np.uint64)
    ix = None if idx is None else _c(idx, np.int64)
    if out.size:
        lib().oracle_move_bits(mode, _ptr(p), None if ix is None else _ptr(ix), _ptr(out), rows, int(n_in), int(n_out), int(shift))
    return out


def flip_bits(packed: np.ndarray, n: int) -> np.ndarray:
    return _move_bits(0, packed, n, n)


def roll_bits(packed: np.ndarray, n: int, shift: int) -> np.ndarray:
    return _move_bits(1, packed, n, n, shift=shift)


def gather_bits(packed: np.ndarray, idx: np.ndarray, n_in: int) -> np.ndarray:
    return _move_bits(2, packed, n_in, int(np.asarray(idx).size), idx=idx)


def scatter_bits(packed: np.ndarray, idx: np.ndarray, src, value: int, n: int) -> np.ndarray:
    """A copy of ``packed`` [..., ceil(n/64)] with bit idx[j] of every row set from bit j of ``src``
    (packed, same leading shape) or, with ``src`` None, from the constant ``value``."""
    out = _u64(packed).copy()
    ix = _c(idx, np.int64)
    rows = int(np.prod(out.shape[:-1], dtype=np.int64)) if out.ndim > 1 else 1
    sp = None if src is None else _u64(src)
    if out.size and ix.size:
        lib().oracle_scatter_bits(_ptr(out), _ptr(ix), None if sp is None else _ptr(sp), int(bool(value)),
                                  rows, int(n), int(ix.size))
    return out
