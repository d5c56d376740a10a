"""The oracle against the reference's golden vectors and against itself.

Pins the C restatement (oracle/brute_oracle.c) to:
  * fixtures produced by the reference's own pure-Python helpers
    (tests/golden/make_golden.py -> golden_ops.npz),
  * the reference's hand-written known-answer vectors,
  * an independent numpy restatement, on seeded random and edge shapes.
"""
import numpy as np
import pytest

from oracle import c_oracle as co
from oracle import np_oracle as no


def test_gemm_golden(golden):
    for idx, (M, K, N) in enumerate(golden["gemm_cases"]):
        a, b = golden[f"gemm{idx}_a"], golden[f"gemm{idx}_b"]
        ap, bp = co.pack_bool(a), co.pack_bool(b)
        assert np.array_equal(ap.view(np.int64), golden[f"gemm{idx}_ap"]), "pack layout differs from LSB-first golden"
        assert np.array_equal(bp.view(np.int64), golden[f"gemm{idx}_bp"])
        c = co.xnor_gemm(ap, bp, int(K))
        assert c.dtype == np.int32 and c.shape == (M, N)
        assert np.array_equal(c, golden[f"gemm{idx}_c"])


def test_popcount_golden(golden):
    for idx in range(int(golden["pop_count"])):
        bits, packed = golden[f"pop{idx}_bits"], golden[f"pop{idx}_packed"]
        assert np.array_equal(co.pack_bool(bits).view(np.int64), packed)
        assert np.array_equal(co.popcount_elems(packed), golden[f"pop{idx}_words"])
        assert co.popcount_total(packed) == int(golden[f"pop{idx}_total"]) == int(bits.sum())
    assert np.array_equal(co.popcount_elems(golden["pop_u8_in"]), golden["pop_u8_out"])
    assert np.array_equal(co.popcount_elems(golden["pop_i32_in"]), golden["pop_i32_out"])


def test_known_answers(golden):
    # float -> bit1 threshold is x > 0 (reference tests/unit/test_dtype.py:79-83)
    x = golden["ka_float_in"]
    assert np.array_equal(co.unpack_bool(co.pack_sign_f32(x, 0), x.shape), golden["ka_float_bits_gt0"])
    # and >= 0 turns the zero on (reference brute/functional.py:131-133)
    assert np.array_equal(co.unpack_bool(co.pack_sign_f32(x, 1), x.shape), [False, True, True, True])
    # unpack_pm1 (reference tests/unit/test_brute_methods.py:92-96)
    bits = golden["ka_pm1_bits"]
    assert np.array_equal(co.unpack_pm1(co.pack_bool(bits), bits.shape), golden["ka_pm1_out"])


def test_not_is_pad_safe(golden):
    rng = np.random.default_rng(7)
    for n in golden["ka_not_sizes"]:
        n = int(n)
        src = rng.integers(0, 2, size=(n,)).astype(bool)
        p = co.pack_bool(src)
        inv = co.bitwise("not", p, None, n)
        assert co.popcount_total(inv) == n - int(src.sum())
        assert np.array_equal(co.unpack_bool(inv, (n,)), ~src)
        assert np.array_equal(inv, no.not_masked(p, n))


SHAPES = [(1,), (5,), (64,), (65,), (3, 13), (13,), (4, 64), (7, 130), (2, 3, 65), (16, 4097)]


@pytest.mark.parametrize("shape", SHAPES)
def test_pack_roundtrip_vs_numpy(shape):
    rng = np.random.default_rng(11)
    x = rng.random(shape) < 0.3
    p = co.pack_bool(x)
    assert np.array_equal(p, no.pack_bool(x))
    assert np.array_equal(co.unpack_bool(p, shape), x)
    assert np.array_equal(co.unpack_pm1(p, shape), no.unpack_pm1(p, shape))
    assert co.popcount_total(p) == int(x.sum())
    assert np.array_equal(co.popcount_elems(p), no.popcount_words(p))
    y = rng.random(shape) < 0.5
    q = co.pack_bool(y)
    assert co.hamming_total(p, q) == int((x ^ y).sum())
    assert np.array_equal(co.hamming_words(p, q), no.popcount_words(p ^ q))
    n = shape[-1]
    assert np.array_equal(co.unpack_bool(co.bitwise("and", p, q, n), shape), x & y)
    assert np.array_equal(co.unpack_bool(co.bitwise("or", p, q, n), shape), x | y)
    assert np.array_equal(co.unpack_bool(co.bitwise("xor", p, q, n), shape), x ^ y)
    assert np.array_equal(co.unpack_bool(co.bitwise("xnor", p, q, n), shape), ~(x ^ y))
    assert co.popcount_total(co.bitwise("xnor", p, q, n)) == int((~(x ^ y)).sum())
    assert np.array_equal(co.unpack_bool(co.bitwise("andnot", p, q, n), shape), x & ~y)
    c = co.pack_bool(rng.random(shape) < 0.5)
    assert np.array_equal(co.select(c, p, q), (p & c) | (q & ~c))
    assert np.array_equal(co.row_any(p), x.any(axis=-1))
    assert np.array_equal(co.row_all(co.bitwise("or", p, co.bitwise("not", p, None, n), n), n),
                          np.ones(shape[:-1], dtype=bool))


def test_empty_and_zero_sizes():
    assert co.pack_bool(np.zeros((3, 0), dtype=bool)).shape == (3, 0)
    assert co.pack_bool(np.zeros((0, 7), dtype=bool)).shape == (0, 1)
    assert co.xnor_gemm(np.zeros((0, 2), np.uint64), np.zeros((5, 2), np.uint64), 128).shape == (0, 5)
    assert co.popcount_total(np.zeros((0,), np.uint64)) == 0


@pytest.mark.parametrize("mode", [0, 1])
def test_pack_sign_vs_numpy(mode):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, 131)).astype(np.float32)
    x[0, :5] = [0.0, -0.0, np.nan, np.inf, -np.inf]
    with np.errstate(invalid="ignore"):
        want = no.pack_bool(no.sign_bits(x, mode))
    assert np.array_equal(co.pack_sign_f32(x, mode), want)


@pytest.mark.parametrize("M,K,N", [(1, 1, 1), (5, 64, 7), (9, 100, 12), (33, 257, 66), (128, 512, 128)])
def test_gemm_vs_pm1_matmul(M, K, N):
    rng = np.random.default_rng(5)
    a = rng.random((M, K)) < 0.5
    b = rng.random((N, K)) < 0.5
    c = co.xnor_gemm(co.pack_bool(a), co.pack_bool(b), K)
    assert np.array_equal(c, no.xnor_gemm(a, b))


def test_config1_checksum():
    # BASELINE config 1 (1024 x 1024 x 4096): the 4x8 blocked path against properties
    rng = np.random.default_rng(1234)
    A = rng.integers(0, 2 ** 63, size=(1024, 64), dtype=np.int64)
    B = rng.integers(0, 2 ** 63, size=(1024, 64), dtype=np.int64)
    C = co.xnor_gemm(A, B, 4096)
    # same parity as K, bounded by K, symmetric under swapping operands
    assert (C % 2 == 0).all() and np.abs(C).max() <= 4096
    assert np.array_equal(co.xnor_gemm(B, A, 4096), C.T)
    # spot rows against the literal definition
    for m in (0, 511, 1023):
        h = no.popcount_words(A[m][None, :] ^ B).sum(axis=-1)
        assert np.array_equal(C[m], 4096 - 2 * h)


def test_mlp_layer_composition():
    rng = np.random.default_rng(9)
    M, K, N = 12, 128, 70
    a = rng.random((M, K)) < 0.5
    w = rng.random((N, K)) < 0.5
    scale = rng.uniform(0.5, 1.5, size=N).astype(np.float32)
    for mode in (0, 1):
        out = co.xnor_gemm_scale_sign_pack(co.pack_bool(a), co.pack_bool(w), scale, K, mode)
        y = no.xnor_gemm(a, w).astype(np.float32) * scale
        assert np.array_equal(out, no.pack_bool(no.sign_bits(y, mode)))


@pytest.mark.parametrize("causal", [True, False])
def test_attention_vs_numpy(causal):
    rng = np.random.default_rng(13)
    B, H, S, D = 1, 2, 48, 128
    q = rng.random((B, H, S, D)) < 0.5
    k = rng.random((B, H, S, D)) < 0.5
    v = rng.standard_normal((B, H, S, D)).astype(np.float32)
    got = co.binary_attention(co.pack_bool(q), co.pack_bool(k), v, causal, D ** -0.5)
    want = no.binary_attention(q, k, v, causal, D ** -0.5)
    assert np.abs(got - want).max() < 1e-5


def test_signed_bundle_vs_numpy():
    # out = sign(sum_n W * pm1(V)), sign(0) = +1, pad bits 0 (reference cbrute/cpu/ops_cpu.cpp:164-213)
    rng = np.random.default_rng(21)
    for B, M, N, D in [(1, 1, 1, 1), (2, 5, 7, 70), (1, 33, 130, 128), (3, 4, 16, 64)]:
        W = rng.integers(-3, 4, size=(B, M, N)).astype(np.int8)
        v = rng.random((B, N, D)) < 0.5
        got = co.signed_bundle(W, co.pack_bool(v), D)
        acc = np.einsum("bmn,bnd->bmd", W.astype(np.int32), np.where(v, 1, -1).astype(np.int32))
        assert np.array_equal(got, no.pack_bool(acc >= 0)), (B, M, N, D)


def test_transpose_bits_vs_numpy():
    rng = np.random.default_rng(31)
    for shape in [(1, 1), (3, 5), (64, 64), (65, 63), (130, 257), (2, 3, 70, 129)]:
        x = rng.random(shape) < 0.5
        got = co.transpose_bits(co.pack_bool(x), shape[-2], shape[-1])
        assert np.array_equal(got, no.pack_bool(np.swapaxes(x, -1, -2))), shape


def test_reduce_rows_vs_numpy():
    rng = np.random.default_rng(32)
    for shape, dim in [((5, 70), 0), ((1, 3), 0), ((4, 6, 130), 1), ((4, 6, 130), 0), ((2, 1, 64), 1)]:
        x = rng.random(shape) < 0.7
        p = co.pack_bool(x)
        assert np.array_equal(co.reduce_rows(p, dim, True), no.pack_bool(x.any(axis=dim))), (shape, dim)
        assert np.array_equal(co.reduce_rows(p, dim, False), no.pack_bool(x.all(axis=dim))), (shape, dim)


def test_move_bits_vs_numpy():
    rng = np.random.default_rng(33)
    for shape in [(1,), (5,), (64,), (65,), (3, 130), (2, 3, 257), (4, 1003)]:
        x = rng.random(shape) < 0.5
        n = shape[-1]
        p = co.pack_bool(x)
        assert np.array_equal(co.flip_bits(p, n), no.pack_bool(np.flip(x, -1))), shape
        for shift in (0, 1, -1, 63, 64, 65, n - 1, n, 3 * n + 7, -2 * n - 5):
            assert np.array_equal(co.roll_bits(p, n, shift), no.pack_bool(np.roll(x, shift, -1))), (shape, shift)
        idx = rng.integers(0, n, size=2 * n + 3)
        assert np.array_equal(co.gather_bits(p, idx, n), no.pack_bool(np.take(x, idx, axis=-1))), shape
