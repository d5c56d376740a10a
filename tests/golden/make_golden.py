"""Generate the golden fixtures in this folder from the REFERENCE's own test helpers.

Run in a checkout where the reference (TheoCoombes/Brute) is available:

    python tests/golden/make_golden.py /path/to/Brute

It imports ``tests/helpers/reference_ops.py`` of the reference (pure-Python,
bit-by-bit implementations that the reference's own tests use as ground truth:
``ref_popcount`` :11-29, ``ref_xnor_popcount_matmul`` :37-62, ``ref_matmul_pm1``
:65-69) and evaluates them on seeded inputs. The reference's compiled extension
cannot be built offline (its Highway submodule is empty), so the packed inputs
are produced by a literal LSB-first packer written here; the reference helpers
then consume those packed words. Also stored: the reference's hand-written
known-answer vectors (tests/unit/test_dtype.py:79-83,
tests/unit/test_brute_methods.py:92-96 and the pad-safe NOT size list :101).

Output: ``golden_ops.npz`` (a few hundred KB). The file is committed; nothing at
test time needs the reference.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch


def load_reference_ops(ref_root: Path):
    path = ref_root / "tests" / "helpers" / "reference_ops.py"
    spec = importlib.util.spec_from_file_location("brute_reference_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def pack_lsb_first(bits: np.ndarray) -> np.ndarray:
    """bool [..., n] -> int64 words, bit i of a row in word i//64 at position i%64."""
    n = bits.shape[-1]
    wpr = (n + 63) // 64
    out = np.zeros(bits.shape[:-1] + (wpr,), dtype=np.uint64)
    for i in range(n):
        out[..., i // 64] |= bits[..., i].astype(np.uint64) << np.uint64(i % 64)
    return out.view(np.int64)


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference>")
    ref_root = Path(sys.argv[1])
    ref = load_reference_ops(ref_root)
    rng = np.random.default_rng(1234)          # the reference's default BRUTE_TEST_SEED
    out = {}

    # GEMM cases: (M, K, N) incl. K not a multiple of 64 (tests/fuzz/test_fuzz_matmul.py:15-34),
    # the parity-catalog shape (4, 64, 4) and one stress shape (64, 1024, 64).
    gemm_cases = [(4, 64, 4), (1, 1, 1), (3, 13, 5), (7, 63, 9), (8, 65, 8), (17, 130, 33),
                  (32, 64, 32), (5, 192, 6), (64, 1024, 64)]
    for idx, (M, K, N) in enumerate(gemm_cases):
        a = rng.integers(0, 2, size=(M, K)).astype(bool)
        b = rng.integers(0, 2, size=(N, K)).astype(bool)
        ap, bp = pack_lsb_first(a), pack_lsb_first(b)
        c_bits = ref.ref_xnor_popcount_matmul(torch.from_numpy(ap), torch.from_numpy(bp), K).numpy()
        c_pm1 = ref.ref_matmul_pm1(torch.from_numpy(a), torch.from_numpy(b).t()).numpy()
        assert np.array_equal(c_bits.astype(np.float32), c_pm1), "reference helpers disagree"
        out[f"gemm{idx}_a"] = a
        out[f"gemm{idx}_b"] = b
        out[f"gemm{idx}_ap"] = ap
        out[f"gemm{idx}_bp"] = bp
        out[f"gemm{idx}_c"] = c_bits.astype(np.int32)
    out["gemm_cases"] = np.array(gemm_cases, dtype=np.int64)

    # per-word popcount of packed buffers (ref_popcount) and totals (ref_packed_popcount)
    pop_shapes = [(8,), (64,), (3, 17), (4, 64), (13,), (3, 13), (2, 1003)]
    for idx, shape in enumerate(pop_shapes):
        bits = rng.integers(0, 2, size=shape).astype(bool)
        packed = pack_lsb_first(bits)
        out[f"pop{idx}_bits"] = bits
        out[f"pop{idx}_packed"] = packed
        out[f"pop{idx}_words"] = ref.ref_popcount(torch.from_numpy(packed)).numpy().astype(np.int32)
        out[f"pop{idx}_total"] = np.int64(ref.ref_packed_popcount(torch.from_numpy(packed)).item())
    out["pop_count"] = np.int64(len(pop_shapes))
    # popcount on narrower dtypes that ref_popcount accepts
    u8 = rng.integers(0, 256, size=(37,), dtype=np.uint8)
    i32 = rng.integers(-2**31, 2**31 - 1, size=(29,), dtype=np.int64).astype(np.int32)
    out["pop_u8_in"] = u8
    out["pop_u8_out"] = ref.ref_popcount(torch.from_numpy(u8)).numpy().astype(np.int32)
    out["pop_i32_in"] = i32
    out["pop_i32_out"] = ref.ref_popcount(torch.from_numpy(i32)).numpy().astype(np.int32)

    # hand-written known answers in the reference's tests
    out["ka_float_in"] = np.array([-1.0, 0.0, 0.5, 1.0], dtype=np.float32)      # test_dtype.py:79-83
    out["ka_float_bits_gt0"] = np.array([False, False, True, True])
    out["ka_pm1_bits"] = np.array([True, False, True, True, False])              # test_brute_methods.py:92-96
    out["ka_pm1_out"] = np.array([1.0, -1.0, 1.0, 1.0, -1.0], dtype=np.float32)
    out["ka_not_sizes"] = np.array([1, 7, 8, 9, 31, 32, 33, 63, 64, 65, 1003, 4096], dtype=np.int64)

    dst = Path(__file__).resolve().parent / "golden_ops.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    main()
