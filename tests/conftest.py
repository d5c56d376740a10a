"""Shared test plumbing.

* ``-m gpu`` tests need a B200; everything else runs on CPU.
* The product registers CUDA kernels only. For the CPU-side tests of the host
  logic (front-end laziness contract, sharding layout) this file binds the CPU
  dispatch key of ``torch.ops.brute.*`` to the ORACLE. That binding exists only
  inside the test process; the package itself never imports the oracle.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = Path(__file__).resolve().parent / "golden" / "golden_ops.npz"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    return np.load(GOLDEN)


@pytest.fixture(scope="session")
def lib_built():
    """Build the CUDA library (nvcc cross-compiles without a GPU) and the oracle."""
    import __graft_entry__ as entry
    entry.build()
    return True


@pytest.fixture
def seed():
    s = int(os.environ.get("BRUTE_TEST_SEED", "1234"))
    torch.manual_seed(s)
    np.random.seed(s % (2 ** 32))
    return s


_CPU_IMPL = None


def install_oracle_cpu_ops():
    """Bind torch.ops.brute.* on the CPU key to the oracle (test process only)."""
    global _CPU_IMPL
    if _CPU_IMPL is not None:
        return
    import brute_b200  # noqa: F401  (defines the schemas)
    from oracle import c_oracle as co

    def t2n(t):
        return t.contiguous().numpy()

    def n2t(a, dtype=None):
        a = np.ascontiguousarray(a)
        if a.dtype == np.uint64:
            a = a.view(np.int64)
        return torch.from_numpy(a)

    def pack_bool(input):
        if input.dim() < 1:
            raise RuntimeError("pack_bool: input must have >= 1 dim")
        if input.dtype != torch.bool:
            raise RuntimeError("pack_bool: input must be torch.bool")
        return n2t(co.pack_bool(t2n(input)), torch.int64)

    def pack_sign(input, mode):
        return n2t(co.pack_sign_f32(t2n(input.float()), mode), torch.int64)

    def unpack_bool(packed, shape):
        shape = [int(s) for s in shape]
        if shape[-1] == 0 or packed.numel() == 0:
            return torch.empty(shape, dtype=torch.bool)
        return torch.from_numpy(co.unpack_bool(t2n(packed), shape))

    def unpack_bits(packed, shape):
        shape = [int(s) for s in shape]
        if shape[-1] == 0 or packed.numel() == 0:
            return torch.empty(shape, dtype=torch.float32)
        return torch.from_numpy(co.unpack_pm1(t2n(packed), shape))

    def gemm(A, B, K):
        if A.dim() != 2 or B.dim() != 2:
            raise RuntimeError("xnor_popcount_matmul: inputs must be 2-D")
        if A.size(1) != B.size(1):
            raise RuntimeError("xnor_popcount_matmul: packed K mismatch")
        return torch.from_numpy(co.xnor_gemm(t2n(A), t2n(B), K))

    def popcount(x):
        return torch.from_numpy(co.popcount_elems(t2n(x)))

    def packed_popcount(x):
        return torch.tensor(co.popcount_total(t2n(x)), dtype=torch.int64)

    def hamming_total(A, B):
        if A.shape != B.shape:
            raise RuntimeError("bit1_hamming_total: shape mismatch")
        return torch.tensor(co.hamming_total(t2n(A), t2n(B)), dtype=torch.int64)

    def not_packed(A, bits):
        if A.numel() == 0:
            return A.clone()
        return n2t(co.bitwise("not", t2n(A), None, bits), torch.int64)

    def bitwise_packed(A, B, op, bits):
        name = {0: "and", 1: "or", 2: "xor", 3: "xnor", 4: "andnot"}[op]
        if A.numel() == 0:
            return A.clone()
        return n2t(co.bitwise(name, t2n(A), t2n(B), bits), torch.int64)

    def mlp(A, B, scale, K, mode):
        return n2t(co.xnor_gemm_scale_sign_pack(t2n(A), t2n(B), t2n(scale), K, mode), torch.int64)

    lib = torch.library.Library("brute", "IMPL", "CPU")
    lib.impl("pack_bool", pack_bool)
    lib.impl("pack_sign", pack_sign)
    lib.impl("unpack_bool", unpack_bool)
    lib.impl("unpack_bits", unpack_bits)
    lib.impl("xnor_popcount_matmul", gemm)
    lib.impl("xnor_popcount_matmul_impl", lambda A, B, K, impl: gemm(A, B, K))
    lib.impl("xnor_popcount_matmul_leave_sms", lambda A, B, K, leave: gemm(A, B, K))
    lib.impl("xnor_matmul_scale_sign_pack", mlp)
    lib.impl("popcount", popcount)
    lib.impl("packed_popcount", packed_popcount)
    lib.impl("bit1_hamming_total", hamming_total)
    lib.impl("hamming_distance", lambda A, B: popcount(torch.bitwise_xor(A, B)))
    lib.impl("bit1_not_packed", not_packed)
    lib.impl("bitwise_packed", bitwise_packed)
    lib.impl("select_packed", lambda c, a, b: n2t(co.select(t2n(c), t2n(a), t2n(b)), torch.int64))
    lib.impl("row_any", lambda A: torch.from_numpy(co.row_any(t2n(A))))
    lib.impl("row_all", lambda A, bits: torch.from_numpy(co.row_all(t2n(A), bits)))

    lib.impl("binary_attention", lambda Qp, Kp, V, causal, scale: torch.from_numpy(
        co.binary_attention(t2n(Qp), t2n(Kp), t2n(V.float()), causal, scale)).to(torch.bfloat16))
    lib.impl("signed_bundle", lambda W, V, D: n2t(co.signed_bundle(t2n(W), t2n(V), D), torch.int64))
    lib.impl("transpose_packed", lambda packed, rows, cols: n2t(co.transpose_bits(t2n(packed.contiguous()), rows, cols), torch.int64))
    lib.impl("flip_packed", lambda packed, n: n2t(co.flip_bits(t2n(packed.contiguous()), n), torch.int64))
    lib.impl("roll_packed", lambda packed, n, shift: n2t(co.roll_bits(t2n(packed.contiguous()), n, shift), torch.int64))
    lib.impl("gather_packed", lambda packed, idx, n_in: n2t(co.gather_bits(t2n(packed.contiguous()), t2n(idx), n_in), torch.int64))
    def scatter_packed_(packed, idx, src, value, n):
        res = co.scatter_bits(t2n(packed), t2n(idx), None if src is None else t2n(src), int(value), n)
        packed.copy_(n2t(res).reshape(packed.shape))
        return packed
    lib.impl("scatter_packed_", scatter_packed_)
    lib.impl("narrow_i32_i16", lambda x: x.to(torch.int16))
    lib.impl("narrow_i32_i16_out", lambda x, out: out.copy_(x.to(torch.int16)))
    lib.impl("xnor_popcount_matmul_out", lambda A, B, K, leave, out: out.copy_(gemm(A, B, K)))

    def unstack_rank_blocks(stacked, out, row0):
        world, rows, n_loc = stacked.shape
        out[row0:row0 + rows] = stacked.permute(1, 0, 2).reshape(rows, world * n_loc).to(torch.int32)
        return out
    lib.impl("unstack_rank_blocks", unstack_rank_blocks)
    lib.impl("reduce_rows_packed", lambda packed, dim, use_or: n2t(co.reduce_rows(t2n(packed.contiguous()), dim, use_or), torch.int64))

    def randomize(out):
        out.random_()
        return out
    lib.impl("randomize_bits", randomize)
    _CPU_IMPL = lib


@pytest.fixture(scope="session")
def cpu_ops(lib_built):
    install_oracle_cpu_ops()
    return True
