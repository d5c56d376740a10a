"""ctypes binding of ``libbrute_b200.so`` (the C ABI declared in include/brute_b200.h).

The library is the only compute path of this package: there is no CPU or eager
fallback. If the shared library is missing the import fails loudly and names
the build command.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libbrute_b200.so"

# keep in step with include/brute_b200.h
OK = 0
UNSUPPORTED = -3        # BRUTE_ERR_UNSUPPORTED: the entry point does not take this shape
ERR_INVALID_ARG, ERR_MISALIGNED, ERR_UNSUPPORTED, ERR_LAUNCH, ERR_WORKSPACE, ERR_DEVICE_WAIT, ERR_DRIVER = -1, -2, -3, -4, -5, -6, -7
SIGN_GT0, SIGN_GE0 = 0, 1
DT_F32, DT_BF16, DT_F16 = 0, 1, 2
OP_AND, OP_OR, OP_XOR, OP_XNOR, OP_ANDNOT = 0, 1, 2, 3, 4
GEMM_AUTO, GEMM_POPC, GEMM_MMA_B1, GEMM_TCGEN05, GEMM_TCGEN05_PAIR = 0, 1, 2, 3, 4

_i64, _p, _i32, _f32 = C.c_int64, C.c_void_p, C.c_int, C.c_float

# name -> argtypes; every function returns int unless listed in _RESTYPES
SIGNATURES = {
    "brute_b200_strerror": [_i32],
    "brute_b200_query_caps": [],
    "brute_b200_device_status": [],
    "brute_b200_selftest_bounded_wait": [_i64, _i32, _p, _p],
    "brute_b200_pack_bool": [_p, _p, _i64, _i64, _p],
    "brute_b200_pack_sign": [_p, _i32, _p, _i64, _i64, _i32, _p],
    "brute_b200_unpack_bool": [_p, _p, _i64, _i64, _p],
    "brute_b200_unpack_pm1_f32": [_p, _p, _i64, _i64, _p],
    "brute_b200_popcount_elems": [_p, _p, _i64, _i32, _p],
    "brute_b200_popcount_total": [_p, _i64, _p, _p],
    "brute_b200_hamming_total": [_p, _p, _i64, _p, _p],
    "brute_b200_hamming_words": [_p, _p, _p, _i64, _p],
    "brute_b200_bitwise": [_i32, _p, _p, _p, _i64, _i64, _i64, _p],
    "brute_b200_not_masked": [_p, _p, _i64, _i64, _i64, _p],
    "brute_b200_select": [_p, _p, _p, _p, _i64, _p],
    "brute_b200_row_any": [_p, _p, _i64, _i64, _p],
    "brute_b200_row_all": [_p, _p, _i64, _i64, _i64, _p],
    "brute_b200_xnor_gemm": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _p],
    "brute_b200_xnor_gemm_leave_sms": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _p],
    "brute_b200_xnor_gemm_scale_sign_pack": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _i32, _p],
    "brute_b200_signed_bundle": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p],
    "brute_b200_signed_bundle_workspace_bytes": [_i64, _i64, _i64],
    "brute_b200_signed_bundle_ws": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p, _i64, _p],
    "brute_b200_signed_bundle_static_max_bytes": [],
    "brute_b200_signed_bundle_static": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _p],
    "brute_b200_transpose_bits": [_p, _p, _i64, _i64, _i64, _p],
    "brute_b200_reduce_rows": [_i32, _p, _p, _i64, _i64, _i64, _p],
    "brute_b200_flip_bits": [_p, _p, _i64, _i64, _p],
    "brute_b200_roll_bits": [_p, _p, _i64, _i64, _i64, _p],
    "brute_b200_gather_bits": [_p, _p, _p, _i64, _i64, _i64, _p],
    "brute_b200_scatter_bits": [_p, _p, _p, _i32, _i64, _i64, _i64, _p],
    "brute_b200_narrow_i32_i16": [_p, _p, _i64, _p],
    "brute_b200_unstack_rank_blocks": [_p, _i32, _p, _i64, _i64, _i64, _i64, _p],
    "brute_b200_xnor_gemm_i16": [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i32, _p],
    "brute_b200_peer_set_flag": [_p, C.c_uint32, _p],
    "brute_b200_peer_wait_flags": [_p, _p, _i32, _i32, _i32, C.c_uint32, _i64, _p],
    "brute_b200_gather_peer_widen": [_p, _p, _p, _i64, _i64, _i32, _i64, _i64, _i32, _i32, _i32, C.c_uint32, _i32, _i64, _p],
    "brute_b200_peer_wait_status": [],
    "brute_b200_binary_attention_fwd": [_p, _p, _p, _p, _i64, _i64, _i64, _i64, _i32, _f32, _p],
}
_RESTYPES = {"brute_b200_strerror": C.c_char_p, "brute_b200_query_caps": C.c_uint32,
             "brute_b200_signed_bundle_workspace_bytes": C.c_int64,
             "brute_b200_signed_bundle_static_max_bytes": C.c_int64}

_lib = None


def load() -> C.CDLL:
    """Load the shared library once and set the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python brute_b200/build.py` (needs nvcc and g++; no GPU required to build)."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.argtypes = argtypes
        fn.restype = _RESTYPES.get(name, C.c_int)
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().brute_b200_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    """Map a negative status to RuntimeError, like TORCH_CHECK in the reference drivers."""
    if code != OK:
        raise RuntimeError(f"{what}: {strerror(code)} (brute_b200 status {code})")
