"""``torch.ops.brute.*`` — the reference's dispatcher namespace, bound to the sm_100a library.

The eleven schemas are the reference's, verbatim (cbrute/ext.cpp:44-66), so any
caller of ``torch.ops.brute.<op>`` keeps working. Each CUDA implementation does
what the reference driver does on the host side (cbrute/cuda/ops_cuda.cu:
validate, make contiguous, allocate the output on the input's device) and then
calls the C ABI on the caller's current stream, inside a device guard (the
reference installs none). Only the CUDA dispatch key is implemented: there is no
CPU kernel and no fallback, an op on a CPU tensor fails in the dispatcher.

Ops beyond the reference's eleven carry new names and never change the eleven:
``pack_sign``, ``bitwise_packed``, ``select_packed``, ``row_any``, ``row_all``,
``xnor_popcount_matmul_impl``, ``xnor_popcount_matmul_leave_sms``, ``xnor_matmul_scale_sign_pack``,
``binary_attention``, ``transpose_packed``, ``reduce_rows_packed``, ``flip_packed``,
``roll_packed``, ``gather_packed``, ``scatter_packed_``, ``narrow_i32_i16``,
``unstack_rank_blocks``. ``signed_bundle`` keeps the reference's schema and
runs on the tensor cores in one launch.
"""
from __future__ import annotations

import os

import torch

from . import _lib as L

_lib = L.load()

_DEF = torch.library.Library("brute", "DEF")

# -- the reference's schemas, verbatim (cbrute/ext.cpp:46-65) -----------------
_DEF.define("pack_bool(Tensor input) -> Tensor")
_DEF.define("unpack_bits(Tensor packed, int[] logical_shape) -> Tensor")
_DEF.define("unpack_bool(Tensor packed, int[] logical_shape) -> Tensor")
_DEF.define("xnor_popcount_matmul(Tensor A, Tensor B, int K) -> Tensor")
_DEF.define("signed_bundle(Tensor W, Tensor V, int D) -> Tensor")
_DEF.define("popcount(Tensor x) -> Tensor")
_DEF.define("packed_popcount(Tensor x) -> Tensor")
_DEF.define("hamming_distance(Tensor A, Tensor B) -> Tensor")
_DEF.define("bit1_hamming_total(Tensor A, Tensor B) -> Tensor")
_DEF.define("bit1_not_packed(Tensor A, int last_dim_bits) -> Tensor")
_DEF.define("randomize_bits(Tensor(a!) out) -> Tensor(a!)")
# -- additions ------------------------------------------------------------------
_DEF.define("pack_sign(Tensor input, int mode) -> Tensor")
_DEF.define("bitwise_packed(Tensor A, Tensor B, int op, int last_dim_bits) -> Tensor")
_DEF.define("select_packed(Tensor cond, Tensor A, Tensor B) -> Tensor")
_DEF.define("row_any(Tensor A) -> Tensor")
_DEF.define("row_all(Tensor A, int last_dim_bits) -> Tensor")
_DEF.define("xnor_popcount_matmul_impl(Tensor A, Tensor B, int K, int impl) -> Tensor")
_DEF.define("xnor_popcount_matmul_leave_sms(Tensor A, Tensor B, int K, int leave_sms) -> Tensor")
_DEF.define("xnor_matmul_scale_sign_pack(Tensor A, Tensor B, Tensor scale, int K, int mode) -> Tensor")
_DEF.define("binary_attention(Tensor Qp, Tensor Kp, Tensor V, bool causal, float scale) -> Tensor")
_DEF.define("transpose_packed(Tensor packed, int rows, int cols) -> Tensor")
_DEF.define("reduce_rows_packed(Tensor packed, int dim, bool use_or) -> Tensor")
_DEF.define("flip_packed(Tensor packed, int n) -> Tensor")
_DEF.define("roll_packed(Tensor packed, int n, int shift) -> Tensor")
_DEF.define("gather_packed(Tensor packed, Tensor idx, int n_in) -> Tensor")
_DEF.define("narrow_i32_i16(Tensor x) -> Tensor")
_DEF.define("narrow_i32_i16_out(Tensor x, Tensor(a!) out) -> Tensor(a!)")
_DEF.define("xnor_popcount_matmul_out(Tensor A, Tensor B, int K, int leave_sms, Tensor(a!) out) -> Tensor(a!)")
_DEF.define("unstack_rank_blocks(Tensor stacked, Tensor(a!) out, int row0) -> Tensor(a!)")
_DEF.define("scatter_packed_(Tensor(a!) packed, Tensor idx, Tensor? src, bool value, int n) -> Tensor(a!)")

_PACK_WIDTH = 64
_SIGN_DTYPES = {torch.float32: L.DT_F32, torch.bfloat16: L.DT_BF16, torch.float16: L.DT_F16}
_POPCOUNT_BYTES = {torch.uint8: 1, torch.bool: 1, torch.int8: 1, torch.int16: 2,
                   torch.int32: 4, torch.int64: 8}


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


_TORCH_CURRENT_STREAM = torch.cuda.current_stream
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_GET_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream(t: torch.Tensor) -> int:
    """The caller's current stream on the tensor's device, as the raw handle the C ABI takes.
    ``torch.cuda.current_stream`` builds a Stream object per call (a few microseconds, on an op
    whose kernel may take as long); the raw handle comes straight from the runtime. Inside a
    ``parallel_streams`` block the op layer has already made the pool stream the real current
    stream (``_rotated``), so the runtime's answer is the right one there too."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(t.device.index)
    return _TORCH_CURRENT_STREAM(t.device).cuda_stream


def _guarded(name: str, fn):
    """What every CUDA implementation gets before its body runs.

    * Every tensor argument must be a CUDA tensor on the first one's device. The dispatcher picks the
      CUDA key as soon as ONE argument is a CUDA tensor and the kernels take raw pointers: a host
      pointer, or another GPU's, would fault the device where ATen and the reference raise.
    * Inside a ``parallel_streams`` block the op runs on the block's next stream (streams.py).
    """
    from . import streams as _streams

    def call(*args):
        dev = None
        for a in args:
            if isinstance(a, torch.Tensor):
                if dev is None:
                    dev = a.device
                    if dev.type != "cuda":
                        raise RuntimeError(f"{name}: expected CUDA tensors, got a tensor on {dev}")
                elif a.device != dev:
                    raise RuntimeError(f"{name}: expected all tensors to be on the same device, "
                                       f"but found at least two devices, {dev} and {a.device}")
        rot = _streams._ACTIVE
        if rot is None:
            return fn(*args)
        return rot.run(fn, args)
    call.__name__ = fn.__name__
    call.__wrapped__ = fn
    return call


class _device_guard:
    """``with torch.cuda.device(dev)`` costs two runtime round trips per op; nearly every call
    is for the device that is current already, where nothing has to be done."""
    __slots__ = ("idx", "prev")

    def __init__(self, device: torch.device):
        self.idx = device.index
        self.prev = -1

    def __enter__(self):
        if self.idx is None:
            return self
        cur = _GET_DEVICE() if _GET_DEVICE is not None else torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


def _words(n_bits: int) -> int:
    return (n_bits + _PACK_WIDTH - 1) // _PACK_WIDTH


# ---------------------------------------------------------------------------
# pack / unpack
# ---------------------------------------------------------------------------
def pack_bool(input: torch.Tensor) -> torch.Tensor:
    _check(input.dim() >= 1, "pack_bool: input must have >= 1 dim")
    _check(input.dtype == torch.bool, "pack_bool: input must be torch.bool")
    inp = input.contiguous()
    ld = inp.size(-1)
    shape = list(inp.shape)
    shape[-1] = _words(ld)
    # every word of the output is written by the kernel: no zero fill needed
    out = torch.empty(shape, dtype=torch.int64, device=inp.device)
    if out.numel() == 0:
        return out
    with _device_guard(inp.device):
        L.check(_lib.brute_b200_pack_bool(inp.data_ptr(), out.data_ptr(), inp.numel() // ld, ld,
                                          _stream(inp)), "pack_bool")
    return out


def pack_sign(input: torch.Tensor, mode: int) -> torch.Tensor:
    _check(input.dim() >= 1, "pack_sign: input must have >= 1 dim")
    _check(input.dtype in _SIGN_DTYPES, "pack_sign: input must be float32, bfloat16 or float16")
    inp = input.contiguous()
    ld = inp.size(-1)
    shape = list(inp.shape)
    shape[-1] = _words(ld)
    out = torch.empty(shape, dtype=torch.int64, device=inp.device)
    if out.numel() == 0:
        return out
    with _device_guard(inp.device):
        L.check(_lib.brute_b200_pack_sign(inp.data_ptr(), _SIGN_DTYPES[inp.dtype], out.data_ptr(),
                                          inp.numel() // ld, ld, int(mode), _stream(inp)), "pack_sign")
    return out


def _unpack_args(packed: torch.Tensor, logical_shape, name: str):
    p = packed.contiguous()
    shape = [int(s) for s in logical_shape]
    _check(len(shape) >= 1, f"{name}: logical_shape must have >= 1 dim")
    return p, shape, shape[-1]


def _unpack_geometry_ok(p: torch.Tensor, shape, ll: int) -> bool:
    rows = 1
    for s in shape[:-1]:
        rows *= s
    return p.size(-1) == _words(ll) and p.numel() == rows * _words(ll)


def unpack_bool(packed: torch.Tensor, logical_shape) -> torch.Tensor:
    p, shape, ll = _unpack_args(packed, logical_shape, "unpack_bool")
    out = torch.empty(shape, dtype=torch.bool, device=p.device)
    if ll == 0 or p.numel() == 0:
        return out
    _check(p.dtype == torch.int64, "unpack_bool: packed must be torch.int64")
    _check(_unpack_geometry_ok(p, shape, ll), "unpack_bool: packed shape does not match logical_shape")
    with _device_guard(p.device):
        L.check(_lib.brute_b200_unpack_bool(p.data_ptr(), out.data_ptr(), p.numel() // p.size(-1), ll,
                                            _stream(p)), "unpack_bool")
    return out


def unpack_bits(packed: torch.Tensor, logical_shape) -> torch.Tensor:
    p, shape, ll = _unpack_args(packed, logical_shape, "unpack_bits")
    out = torch.empty(shape, dtype=torch.float32, device=p.device)
    if ll == 0 or p.numel() == 0:
        return out
    _check(p.dtype == torch.int64, "unpack_bits: packed must be torch.int64")
    _check(_unpack_geometry_ok(p, shape, ll), "unpack_bits: packed shape does not match logical_shape")
    with _device_guard(p.device):
        L.check(_lib.brute_b200_unpack_pm1_f32(p.data_ptr(), out.data_ptr(), p.numel() // p.size(-1), ll,
                                               _stream(p)), "unpack_bits")
    return out


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def _gemm_args(A: torch.Tensor, B: torch.Tensor, K: int, name: str):
    _check(A.dim() == 2 and B.dim() == 2, f"{name}: inputs must be 2-D")
    _check(A.size(1) == B.size(1), f"{name}: packed K mismatch")
    _check(A.dtype == torch.int64 and B.dtype == torch.int64, f"{name}: inputs must be int64 packed buffers")
    _check(A.device == B.device, f"{name}: inputs must be on the same device")
    _check(0 <= int(K) <= 64 * A.size(1), f"{name}: K out of range for the packed width")
    return A.contiguous(), B.contiguous()


def xnor_popcount_matmul_impl(A: torch.Tensor, B: torch.Tensor, K: int, impl: int) -> torch.Tensor:
    Ac, Bc = _gemm_args(A, B, K, "xnor_popcount_matmul")
    M, N, Kp = Ac.size(0), Bc.size(0), Ac.size(1)
    C = torch.empty((M, N), dtype=torch.int32, device=Ac.device)
    if M == 0 or N == 0:
        return C
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_xnor_gemm(Ac.data_ptr(), Bc.data_ptr(), C.data_ptr(), M, N, Kp, int(K), N,
                                          int(impl), _stream(Ac)), "xnor_popcount_matmul")
    return C


def xnor_popcount_matmul(A: torch.Tensor, B: torch.Tensor, K: int) -> torch.Tensor:
    return xnor_popcount_matmul_impl(A, B, K, L.GEMM_AUTO)


def xnor_popcount_matmul_leave_sms(A: torch.Tensor, B: torch.Tensor, K: int, leave_sms: int) -> torch.Tensor:
    """The same GEMM with `leave_sms` SMs left free for kernels of other streams (a collective)."""
    Ac, Bc = _gemm_args(A, B, K, "xnor_popcount_matmul")
    M, N, Kp = Ac.size(0), Bc.size(0), Ac.size(1)
    C = torch.empty((M, N), dtype=torch.int32, device=Ac.device)
    if M == 0 or N == 0:
        return C
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_xnor_gemm_leave_sms(Ac.data_ptr(), Bc.data_ptr(), C.data_ptr(), M, N, Kp, int(K), N,
                                                    int(leave_sms), _stream(Ac)), "xnor_popcount_matmul")
    return C


def xnor_matmul_scale_sign_pack(A, B, scale, K: int, mode: int) -> torch.Tensor:
    Ac, Bc = _gemm_args(A, B, K, "xnor_matmul_scale_sign_pack")
    M, N, Kp = Ac.size(0), Bc.size(0), Ac.size(1)
    _check(scale.dtype == torch.float32 and scale.numel() == N and scale.device == Ac.device,
           "xnor_matmul_scale_sign_pack: scale must be float32 [N] on the inputs' device")
    sc = scale.contiguous()
    out = torch.empty((M, _words(N)), dtype=torch.int64, device=Ac.device)
    if out.numel() == 0:
        return out
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_xnor_gemm_scale_sign_pack(
            Ac.data_ptr(), Bc.data_ptr(), sc.data_ptr(), out.data_ptr(), M, N, Kp, int(K), int(mode),
            L.GEMM_AUTO, _stream(Ac)), "xnor_matmul_scale_sign_pack")
    return out


def signed_bundle(W: torch.Tensor, V: torch.Tensor, D: int) -> torch.Tensor:
    _check(W.dim() == 3 and V.dim() == 3, "signed_bundle: W (B,M,N), V packed (B,N,Dp)")
    _check(W.dtype == torch.int8, "signed_bundle: W must be int8")
    B, M, N = W.shape
    Dp = V.size(2)
    _check(V.size(0) == B and V.size(1) == N, "signed_bundle: W (B,M,N) / V (B,N,Dp) batch or N mismatch")
    _check(V.dtype == torch.int64 and 0 <= int(D) <= 64 * Dp, "signed_bundle: V must be int64 packed with D <= 64*Dp")
    Wc, Vc = W.contiguous(), V.contiguous()
    out = torch.empty((B, M, Dp), dtype=torch.int64, device=V.device)
    if out.numel():
        with _device_guard(V.device):
            # one launch, no scratch: the tensor-core kernel transposes V's bit blocks itself
            L.check(_lib.brute_b200_signed_bundle(Wc.data_ptr() if Wc.numel() else None,
                                                  Vc.data_ptr() if Vc.numel() else None, out.data_ptr(),
                                                  B, M, N, Dp, int(D), _stream(V)), "signed_bundle")
    return out


# ---------------------------------------------------------------------------
# popcount / hamming
# ---------------------------------------------------------------------------
def popcount(x: torch.Tensor) -> torch.Tensor:
    p = x.contiguous()
    _check(p.dtype in _POPCOUNT_BYTES, f"popcount: unsupported dtype {p.dtype}")
    out = torch.empty(p.shape, dtype=torch.int32, device=p.device)
    if p.numel() == 0:
        return out
    with _device_guard(p.device):
        L.check(_lib.brute_b200_popcount_elems(p.data_ptr(), out.data_ptr(), p.numel(),
                                               _POPCOUNT_BYTES[p.dtype], _stream(p)), "popcount")
    return out


def packed_popcount(x: torch.Tensor) -> torch.Tensor:
    p = x.contiguous()
    out = torch.empty((), dtype=torch.int64, device=p.device)      # overwritten by the call itself
    with _device_guard(p.device):
        L.check(_lib.brute_b200_popcount_total(p.data_ptr() if p.numel() else None,
                                               p.numel() * p.element_size(), out.data_ptr(), _stream(p)),
                "packed_popcount")
    return out


def bit1_hamming_total(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    _check(A.shape == B.shape, "bit1_hamming_total: shape mismatch")
    _check(A.dtype == B.dtype, "bit1_hamming_total: dtype mismatch")
    Ac, Bc = A.contiguous(), B.contiguous()
    out = torch.empty((), dtype=torch.int64, device=Ac.device)
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_hamming_total(Ac.data_ptr() if Ac.numel() else None,
                                              Bc.data_ptr() if Bc.numel() else None,
                                              Ac.numel() * Ac.element_size(), out.data_ptr(), _stream(Ac)),
                "bit1_hamming_total")
    return out


def hamming_distance(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    if A.shape == B.shape and A.dtype == torch.int64 and B.dtype == torch.int64:
        Ac, Bc = A.contiguous(), B.contiguous()
        out = torch.empty(Ac.shape, dtype=torch.int32, device=Ac.device)
        if Ac.numel():
            with _device_guard(Ac.device):
                L.check(_lib.brute_b200_hamming_words(Ac.data_ptr(), Bc.data_ptr(), out.data_ptr(),
                                                      Ac.numel(), _stream(Ac)), "hamming_distance")
        return out
    return popcount(torch.bitwise_xor(A, B))       # broadcasting / other dtypes


# ---------------------------------------------------------------------------
# bitwise
# ---------------------------------------------------------------------------
def bit1_not_packed(A: torch.Tensor, last_dim_bits: int) -> torch.Tensor:
    _check(A.dtype == torch.int64, "bit1_not_packed: input must be int64")
    Ac = A.contiguous()
    out = torch.empty_like(Ac)
    if Ac.numel() == 0:
        return out
    wpr = Ac.size(-1) if Ac.dim() else 1
    # the reference leaves the tail alone when last_dim_bits == 0 or a multiple of 64
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_not_masked(Ac.data_ptr(), out.data_ptr(), Ac.numel() // wpr, wpr,
                                           int(last_dim_bits), _stream(Ac)), "bit1_not_packed")
    return out


def bitwise_packed(A: torch.Tensor, B: torch.Tensor, op: int, last_dim_bits: int) -> torch.Tensor:
    _check(A.shape == B.shape, "bitwise_packed: shape mismatch")
    _check(A.dtype == torch.int64 and B.dtype == torch.int64, "bitwise_packed: inputs must be int64")
    Ac, Bc = A.contiguous(), B.contiguous()
    out = torch.empty_like(Ac)
    if Ac.numel() == 0:
        return out
    wpr = Ac.size(-1) if Ac.dim() else 1
    with _device_guard(Ac.device):
        L.check(_lib.brute_b200_bitwise(int(op), Ac.data_ptr(), Bc.data_ptr(), out.data_ptr(),
                                        Ac.numel() // wpr, wpr, int(last_dim_bits), _stream(Ac)),
                "bitwise_packed")
    return out


def select_packed(cond: torch.Tensor, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    _check(cond.shape == A.shape == B.shape, "select_packed: shape mismatch")
    c, a, b = cond.contiguous(), A.contiguous(), B.contiguous()
    out = torch.empty_like(a)
    if a.numel():
        with _device_guard(a.device):
            L.check(_lib.brute_b200_select(c.data_ptr(), a.data_ptr(), b.data_ptr(), out.data_ptr(),
                                           a.numel(), _stream(a)), "select_packed")
    return out


def row_any(A: torch.Tensor) -> torch.Tensor:
    _check(A.dim() >= 1 and A.dtype == torch.int64, "row_any: input must be int64 with >= 1 dim")
    Ac = A.contiguous()
    out = torch.empty(Ac.shape[:-1], dtype=torch.bool, device=Ac.device)
    if out.numel():
        with _device_guard(Ac.device):
            L.check(_lib.brute_b200_row_any(Ac.data_ptr() if Ac.numel() else None, out.data_ptr(),
                                            out.numel(), Ac.size(-1), _stream(Ac)), "row_any")
    return out


def row_all(A: torch.Tensor, last_dim_bits: int) -> torch.Tensor:
    _check(A.dim() >= 1 and A.dtype == torch.int64, "row_all: input must be int64 with >= 1 dim")
    Ac = A.contiguous()
    out = torch.empty(Ac.shape[:-1], dtype=torch.bool, device=Ac.device)
    if out.numel():
        with _device_guard(Ac.device):
            L.check(_lib.brute_b200_row_all(Ac.data_ptr() if Ac.numel() else None, out.data_ptr(),
                                            out.numel(), Ac.size(-1), int(last_dim_bits), _stream(Ac)),
                    "row_all")
    return out


def transpose_packed(packed: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    """packed [..., rows, ceil(cols/64)] -> packed [..., cols, ceil(rows/64)]: the bit matrices transposed."""
    _check(packed.dim() >= 2 and packed.dtype == torch.int64, "transpose_packed: input must be int64 with >= 2 dims")
    rows, cols = int(rows), int(cols)
    _check(packed.size(-2) == rows and packed.size(-1) == _words(cols),
           "transpose_packed: packed shape must be [..., rows, ceil(cols/64)]")
    pc = packed.contiguous()
    batch = 1
    for d in pc.shape[:-2]:
        batch *= int(d)
    out = torch.empty(tuple(pc.shape[:-2]) + (cols, _words(rows)), dtype=torch.int64, device=pc.device)
    if out.numel():
        with _device_guard(pc.device):
            L.check(_lib.brute_b200_transpose_bits(pc.data_ptr(), out.data_ptr(), batch, rows, cols, _stream(pc)),
                    "transpose_packed")
    return out


def reduce_rows_packed(packed: torch.Tensor, dim: int, use_or: bool) -> torch.Tensor:
    """OR (any) or AND (all) over a non-packed dimension of a packed buffer, in one pass."""
    _check(packed.dtype == torch.int64 and packed.dim() >= 2, "reduce_rows_packed: input must be int64 with >= 2 dims")
    nd = packed.dim()
    d = int(dim) if int(dim) >= 0 else nd + int(dim)
    _check(0 <= d < nd - 1, "reduce_rows_packed: dim must be a non-packed dimension")
    pc = packed.contiguous()
    outer = 1
    for s_ in pc.shape[:d]:
        outer *= int(s_)
    inner = 1
    for s_ in pc.shape[d + 1:]:
        inner *= int(s_)
    out = torch.empty(tuple(pc.shape[:d]) + tuple(pc.shape[d + 1:]), dtype=torch.int64, device=pc.device)
    if out.numel():
        with _device_guard(pc.device):
            L.check(_lib.brute_b200_reduce_rows(L.OP_OR if use_or else L.OP_AND, pc.data_ptr() if pc.numel() else None,
                                                out.data_ptr(), outer, int(pc.size(d)), inner, _stream(pc)),
                    "reduce_rows_packed")
    return out


def _packed_rows(packed: torch.Tensor, n: int, what: str):
    _check(packed.dim() >= 1 and packed.dtype == torch.int64, f"{what}: input must be int64 with >= 1 dim")
    _check(packed.size(-1) == _words(int(n)), f"{what}: last dimension must be ceil(n/64) words")
    pc = packed.contiguous()
    rows = pc.numel() // pc.size(-1) if pc.size(-1) else 0
    return pc, rows


def flip_packed(packed: torch.Tensor, n: int) -> torch.Tensor:
    """Reverse the n bits of every row of a packed buffer (flip along the packed axis)."""
    pc, rows = _packed_rows(packed, n, "flip_packed")
    out = torch.empty_like(pc)
    if out.numel():
        with _device_guard(pc.device):
            L.check(_lib.brute_b200_flip_bits(pc.data_ptr(), out.data_ptr(), rows, int(n), _stream(pc)), "flip_packed")
    return out


def roll_packed(packed: torch.Tensor, n: int, shift: int) -> torch.Tensor:
    """torch.roll along the packed axis: out bit j = in bit (j - shift) mod n."""
    pc, rows = _packed_rows(packed, n, "roll_packed")
    out = torch.empty_like(pc)
    if out.numel():
        with _device_guard(pc.device):
            L.check(_lib.brute_b200_roll_bits(pc.data_ptr(), out.data_ptr(), rows, int(n), int(shift), _stream(pc)),
                    "roll_packed")
    return out


def gather_packed(packed: torch.Tensor, idx: torch.Tensor, n_in: int) -> torch.Tensor:
    """index_select along the packed axis: out bit j of every row = in bit idx[j]."""
    pc, rows = _packed_rows(packed, n_in, "gather_packed")
    _check(idx.dim() == 1 and idx.dtype == torch.int64 and idx.device == pc.device,
           "gather_packed: idx must be a 1-D int64 tensor on the input's device")
    ic = idx.contiguous()
    n_out = int(ic.numel())
    out = torch.empty(tuple(pc.shape[:-1]) + (_words(n_out),), dtype=torch.int64, device=pc.device)
    if out.numel():
        with _device_guard(pc.device):
            L.check(_lib.brute_b200_gather_bits(pc.data_ptr() if pc.numel() else None, ic.data_ptr(), out.data_ptr(),
                                                rows if pc.size(-1) else out.numel() // out.size(-1), int(n_in), n_out,
                                                _stream(pc)), "gather_packed")
    return out


def scatter_packed_(packed: torch.Tensor, idx: torch.Tensor, src, value: bool, n: int) -> torch.Tensor:
    """In place: bit idx[j] of every row of ``packed`` = bit j of the row of ``src`` (packed), or ``value``."""
    _check(packed.dim() >= 1 and packed.dtype == torch.int64 and packed.is_contiguous(),
           "scatter_packed_: packed must be a contiguous int64 tensor with >= 1 dim")
    _check(packed.size(-1) == _words(int(n)), "scatter_packed_: last dimension must be ceil(n/64) words")
    _check(idx.dim() == 1 and idx.dtype == torch.int64, "scatter_packed_: idx must be a 1-D int64 tensor")
    ic = idx.contiguous()
    n_idx = int(ic.numel())
    rows = packed.numel() // packed.size(-1) if packed.size(-1) else 0
    sc = None
    if src is not None:
        _check(src.dtype == torch.int64 and tuple(src.shape) == tuple(packed.shape[:-1]) + (_words(n_idx),),
               "scatter_packed_: src must be int64 packed [..., ceil(len(idx)/64)] with packed's leading shape")
        sc = src.contiguous()
    if rows and n_idx:
        with _device_guard(packed.device):
            L.check(_lib.brute_b200_scatter_bits(packed.data_ptr(), ic.data_ptr(), sc.data_ptr() if sc is not None else None,
                                                 int(bool(value)), rows, int(n), n_idx, _stream(packed)), "scatter_packed_")
    return packed


def narrow_i32_i16(x: torch.Tensor) -> torch.Tensor:
    """int32 -> int16, exact for |v| <= 32767: the transport form of a GEMM block with K <= 32767."""
    _check(x.dtype == torch.int32, "narrow_i32_i16: input must be int32")
    xc = x.contiguous()
    out = torch.empty(xc.shape, dtype=torch.int16, device=xc.device)
    if xc.numel():
        with _device_guard(xc.device):
            L.check(_lib.brute_b200_narrow_i32_i16(xc.data_ptr(), out.data_ptr(), xc.numel(), _stream(xc)), "narrow_i32_i16")
    return out


def narrow_i32_i16_out(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _check(x.dtype == torch.int32 and out.dtype == torch.int16 and x.is_contiguous() and out.is_contiguous()
           and x.numel() == out.numel(), "narrow_i32_i16_out: contiguous int32 input and int16 output of one size")
    if x.numel():
        with _device_guard(x.device):
            L.check(_lib.brute_b200_narrow_i32_i16(x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)), "narrow_i32_i16")
    return out


def xnor_popcount_matmul_out(A: torch.Tensor, B: torch.Tensor, K: int, leave_sms: int, out: torch.Tensor) -> torch.Tensor:
    """The GEMM into a caller-provided contiguous int32 [M, N] tensor (no allocation in the call)."""
    Ac, Bc = _gemm_args(A, B, K, "xnor_popcount_matmul")
    M, N, Kp = Ac.size(0), Bc.size(0), Ac.size(1)
    _check(out.dtype == torch.int32 and tuple(out.shape) == (M, N) and out.is_contiguous(),
           "xnor_popcount_matmul_out: out must be a contiguous int32 [M, N] tensor")
    if M and N:
        with _device_guard(Ac.device):
            L.check(_lib.brute_b200_xnor_gemm_leave_sms(Ac.data_ptr(), Bc.data_ptr(), out.data_ptr(), M, N, Kp, int(K), N,
                                                        int(leave_sms), _stream(Ac)), "xnor_popcount_matmul")
    return out


def unstack_rank_blocks(stacked: torch.Tensor, out: torch.Tensor, row0: int) -> torch.Tensor:
    """stacked [world, rows, n_loc] (int16 or int32: what an all-gather of the rank blocks delivers)
    -> out[row0 : row0 + rows, :] of the row-major int32 result [M, world * n_loc], in place."""
    _check(stacked.dim() == 3 and stacked.dtype in (torch.int16, torch.int32) and stacked.is_contiguous(),
           "unstack_rank_blocks: stacked must be a contiguous int16/int32 [world, rows, n_loc] tensor")
    world, rows, n_loc = (int(v) for v in stacked.shape)
    _check(out.dim() == 2 and out.dtype == torch.int32 and out.is_contiguous() and out.size(1) == world * n_loc,
           "unstack_rank_blocks: out must be a contiguous int32 [M, world * n_loc] tensor")
    row0 = int(row0)
    _check(0 <= row0 and row0 + rows <= out.size(0), "unstack_rank_blocks: rows out of range")
    if stacked.numel():
        with _device_guard(out.device):
            L.check(_lib.brute_b200_unstack_rank_blocks(stacked.data_ptr(), stacked.element_size(),
                                                        out.data_ptr() + row0 * out.size(1) * 4, world, rows, n_loc,
                                                        out.size(1), _stream(out)), "unstack_rank_blocks")
    return out


def randomize_bits(out: torch.Tensor) -> torch.Tensor:
    out.random_()          # cbrute/cuda/ops_cuda.cu:340, a plain ATen call
    return out


# ---------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------
def binary_attention(Qp: torch.Tensor, Kp: torch.Tensor, V: torch.Tensor, causal: bool, scale: float) -> torch.Tensor:
    _check(V.dim() == 4 and Qp.dim() == 4 and Kp.dim() == 4, "binary_attention: Qp, Kp, V must be 4-D [B,H,S,*]")
    B, H, S, D = V.shape
    _check(V.dtype == torch.bfloat16, "binary_attention: V must be bfloat16")
    _check(Qp.dtype == torch.int64 and Kp.dtype == torch.int64, "binary_attention: Qp, Kp must be int64 packed")
    _check(D in (64, 128), "binary_attention: head dim must be 64 or 128")
    _check(tuple(Qp.shape) == (B, H, S, D // 64) and tuple(Kp.shape) == (B, H, S, D // 64),
           "binary_attention: packed Q/K shape must be [B,H,S,D/64]")
    q, k, v = Qp.contiguous(), Kp.contiguous(), V.contiguous()
    out = torch.empty_like(v)
    if out.numel():
        with _device_guard(v.device):
            L.check(_lib.brute_b200_binary_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                                         B, H, S, D, int(bool(causal)), float(scale), _stream(v)),
                    "binary_attention")
    return out


_CUDA_IMPLS = {
    "pack_bool": pack_bool, "unpack_bits": unpack_bits, "unpack_bool": unpack_bool,
    "xnor_popcount_matmul": xnor_popcount_matmul, "signed_bundle": signed_bundle,
    "popcount": popcount, "packed_popcount": packed_popcount, "hamming_distance": hamming_distance,
    "bit1_hamming_total": bit1_hamming_total, "bit1_not_packed": bit1_not_packed,
    "randomize_bits": randomize_bits,
    "pack_sign": pack_sign, "bitwise_packed": bitwise_packed, "select_packed": select_packed,
    "row_any": row_any, "row_all": row_all, "xnor_popcount_matmul_impl": xnor_popcount_matmul_impl,
    "xnor_popcount_matmul_leave_sms": xnor_popcount_matmul_leave_sms,
    "xnor_matmul_scale_sign_pack": xnor_matmul_scale_sign_pack, "binary_attention": binary_attention,
    "transpose_packed": transpose_packed, "reduce_rows_packed": reduce_rows_packed,
    "flip_packed": flip_packed, "roll_packed": roll_packed, "gather_packed": gather_packed,
    "scatter_packed_": scatter_packed_, "narrow_i32_i16": narrow_i32_i16, "unstack_rank_blocks": unstack_rank_blocks,
    "narrow_i32_i16_out": narrow_i32_i16_out, "xnor_popcount_matmul_out": xnor_popcount_matmul_out,
}
# Two bindings of the CUDA dispatch key to the same C ABI, chosen by BRUTE_B200_BINDING at import:
#   "cpp"     (default) the compiled functions of csrc_host/cbrute.cpp, the layer the reference has in
#             cbrute/ext.cpp + cbrute/cuda/ops_cuda.cu: no Python between the dispatcher and the
#             launch (6.4-7.5 us of host time per op against 11.4-14.7 us through ctypes). They ask
#             the runtime for the current stream, as the reference's do, so inside a
#             ``parallel_streams`` block they stay on the caller's stream;
#   "ctypes"  the Python functions above, through ctypes: the binding whose ops rotate over the pool
#             streams of ``parallel_streams``, and the one to read when following a call.
BINDING = os.environ.get("BRUTE_B200_BINDING", "cpp").strip().lower() or "cpp"
if BINDING not in ("cpp", "ctypes"):
    raise ImportError(f"BRUTE_B200_BINDING must be 'cpp' or 'ctypes', got {BINDING!r}")
_IMPL = None
if BINDING == "cpp":
    from . import _cbrute
    _cbrute.register_cuda_ops()
else:
    _IMPL = torch.library.Library("brute", "IMPL", "CUDA")
    for _name, _fn in _CUDA_IMPLS.items():
        _IMPL.impl(_name, _guarded(_name, _fn))


# Shape-only kernels so that FakeTensor / torch.compile tracing sees the ops
# (the reference registers none and graph-breaks).
def _register_fakes() -> None:
    reg = torch.library.register_fake

    def packed_like(x):
        s = list(x.shape)
        s[-1] = _words(s[-1])
        return x.new_empty(s, dtype=torch.int64)

    reg("brute::pack_bool")(lambda input: packed_like(input))
    reg("brute::pack_sign")(lambda input, mode: packed_like(input))
    reg("brute::unpack_bool")(lambda packed, logical_shape: packed.new_empty(list(logical_shape), dtype=torch.bool))
    reg("brute::unpack_bits")(lambda packed, logical_shape: packed.new_empty(list(logical_shape), dtype=torch.float32))
    reg("brute::xnor_popcount_matmul")(lambda A, B, K: A.new_empty((A.shape[0], B.shape[0]), dtype=torch.int32))
    reg("brute::xnor_popcount_matmul_leave_sms")(lambda A, B, K, leave_sms: A.new_empty((A.shape[0], B.shape[0]), dtype=torch.int32))
    reg("brute::xnor_popcount_matmul_impl")(lambda A, B, K, impl: A.new_empty((A.shape[0], B.shape[0]), dtype=torch.int32))
    reg("brute::xnor_matmul_scale_sign_pack")(
        lambda A, B, scale, K, mode: A.new_empty((A.shape[0], _words(B.shape[0])), dtype=torch.int64))
    reg("brute::popcount")(lambda x: x.new_empty(x.shape, dtype=torch.int32))
    reg("brute::packed_popcount")(lambda x: x.new_empty((), dtype=torch.int64))
    reg("brute::bit1_hamming_total")(lambda A, B: A.new_empty((), dtype=torch.int64))
    reg("brute::hamming_distance")(lambda A, B: torch.empty_like(torch.bitwise_xor(A, B), dtype=torch.int32))
    reg("brute::bit1_not_packed")(lambda A, last_dim_bits: torch.empty_like(A))
    reg("brute::bitwise_packed")(lambda A, B, op, last_dim_bits: torch.empty_like(A))
    reg("brute::select_packed")(lambda cond, A, B: torch.empty_like(A))
    reg("brute::row_any")(lambda A: A.new_empty(A.shape[:-1], dtype=torch.bool))
    reg("brute::row_all")(lambda A, last_dim_bits: A.new_empty(A.shape[:-1], dtype=torch.bool))
    reg("brute::signed_bundle")(lambda W, V, D: V.new_empty((W.shape[0], W.shape[1], V.shape[2]), dtype=torch.int64))
    reg("brute::binary_attention")(lambda Qp, Kp, V, causal, scale: torch.empty_like(V))
    reg("brute::transpose_packed")(
        lambda packed, rows, cols: packed.new_empty(tuple(packed.shape[:-2]) + (cols, _words(rows)), dtype=torch.int64))
    reg("brute::flip_packed")(lambda packed, n: torch.empty_like(packed))
    reg("brute::roll_packed")(lambda packed, n, shift: torch.empty_like(packed))
    reg("brute::gather_packed")(
        lambda packed, idx, n_in: packed.new_empty(tuple(packed.shape[:-1]) + (_words(idx.shape[0]),), dtype=torch.int64))
    reg("brute::narrow_i32_i16")(lambda x: torch.empty_like(x, dtype=torch.int16))
    reg("brute::narrow_i32_i16_out")(lambda x, out: out)
    reg("brute::xnor_popcount_matmul_out")(lambda A, B, K, leave_sms, out: out)
    reg("brute::unstack_rank_blocks")(lambda stacked, out, row0: out)
    reg("brute::scatter_packed_")(lambda packed, idx, src, value, n: packed)
    reg("brute::reduce_rows_packed")(
        lambda packed, dim, use_or: packed.new_empty(tuple(s for i, s in enumerate(packed.shape) if i != dim % packed.dim()),
                                                     dtype=torch.int64))


try:
    _register_fakes()
except Exception:       # older torch without register_fake: tracing support is optional
    pass
