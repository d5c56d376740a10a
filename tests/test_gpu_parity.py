"""GPU parity: every kernel, called through torch.ops.brute.* -> ctypes -> the C ABI,
against the CPU oracle on the same seeded inputs (bit-exact for integer work),
against the committed golden fixtures, and through size-independent properties
at the full BASELINE sizes."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ops(lib_built):
    import brute_b200  # noqa: F401
    return torch.ops.brute


@pytest.fixture(scope="module")
def co():
    from oracle import c_oracle
    return c_oracle


def u64(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy().view(np.uint64)


def gen(seed):
    return torch.Generator(device="cpu").manual_seed(seed)


# ---------------------------------------------------------------------------
# pack / unpack
# ---------------------------------------------------------------------------
TAIL_SHAPES = [(n,) for n in list(range(1, 131)) + [191, 192, 193, 255, 256, 257, 1003, 4096, 4097]]
ND_SHAPES = [(3, 13), (13,), (4, 64), (7, 130), (2, 3, 65), (33, 1003), (5, 4097), (256, 4097),
             (1, 1), (1, 65536), (65537,), (17, 16), (1000, 7), (9, 48), (6, 80),
             (3, 32), (5, 33), (4, 8), (11, 9), (2, 31), (129, 95), (64, 63), (2, 4099)]


@pytest.mark.parametrize("shape", TAIL_SHAPES[::3] + ND_SHAPES)
def test_pack_unpack_bool(ops, co, shape):
    x = torch.rand(shape, generator=gen(sum(shape))) < 0.3
    p = ops.pack_bool(x.to(DEV))
    assert p.dtype == torch.int64 and tuple(p.shape) == shape[:-1] + ((shape[-1] + 63) // 64,)
    assert np.array_equal(u64(p), co.pack_bool(x.numpy()))
    assert torch.equal(ops.unpack_bool(p, list(shape)).cpu(), x)
    assert np.array_equal(ops.unpack_bits(p, list(shape)).cpu().numpy(), co.unpack_pm1(u64(p), shape))
    assert int(ops.packed_popcount(p)) == int(x.sum())


def test_pack_bool_any_nonzero_byte_is_one(ops, co):
    raw = torch.randint(0, 256, (37, 201), generator=gen(1), dtype=torch.uint8)
    raw[raw < 128] = 0
    x = raw.view(torch.bool)
    assert np.array_equal(u64(ops.pack_bool(x.to(DEV))), co.pack_bool(raw.numpy()))


def test_pack_bool_unaligned_base(ops, co):
    # a view that starts 1..15 bytes into an allocation: rows and base both unaligned
    big = torch.rand((70000,), generator=gen(2)) < 0.5
    d = big.to(DEV)
    for off in (1, 3, 8, 15):
        for n in (64 * 100, 4097, 999):
            v = d[off:off + n]
            assert v.data_ptr() % 16 != 0 or off % 16 == 0
            got = ops.pack_bool(v)      # .contiguous() is a no-op on a 1-D slice: the offset survives
            assert np.array_equal(u64(got), co.pack_bool(big[off:off + n].numpy()))
            assert torch.equal(ops.unpack_bool(got, [n]).cpu(), big[off:off + n])


def test_pack_empty_and_ragged(ops):
    assert tuple(ops.pack_bool(torch.zeros((3, 0), dtype=torch.bool, device=DEV)).shape) == (3, 0)
    assert tuple(ops.pack_bool(torch.zeros((0, 7), dtype=torch.bool, device=DEV)).shape) == (0, 1)
    assert tuple(ops.unpack_bool(torch.zeros((0, 1), dtype=torch.int64, device=DEV), [0, 7]).shape) == (0, 7)
    with pytest.raises(RuntimeError, match="must be torch.bool"):
        ops.pack_bool(torch.zeros(4, device=DEV))
    with pytest.raises(RuntimeError, match=">= 1 dim"):
        ops.pack_bool(torch.zeros((), dtype=torch.bool, device=DEV))


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("shape", [(1,), (63,), (64,), (65,), (9, 131), (3, 256), (5, 4097), (1 << 16,), (31, 1003)])
def test_pack_sign_f32(ops, co, mode, shape):
    x = torch.randn(shape, generator=gen(mode + sum(shape)))
    flat = x.view(-1)
    flat[: min(5, flat.numel())] = torch.tensor([0.0, -0.0, float("nan"), float("inf"), -float("inf")])[: min(5, flat.numel())]
    assert np.array_equal(u64(ops.pack_sign(x.to(DEV), mode)), co.pack_sign_f32(x.numpy(), mode))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(1,), (65,), (9, 131), (9, 130), (4, 512), (1 << 15,), (3, 1003)])
def test_pack_sign_16bit(ops, co, dtype, shape):
    x = torch.randn(shape, generator=gen(sum(shape))).to(dtype)
    x.view(-1)[0] = 0.0
    for mode in (0, 1):
        assert np.array_equal(u64(ops.pack_sign(x.to(DEV), mode)), co.pack_sign_f32(x.float().numpy(), mode))


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("k", [20, 24, 27])
def test_pack_sign_f32_at_sweep_sizes(ops, co, mode, k):
    """The pack sweep of the benchmark configuration (fp32 [2^k], N(0,1), k = 10..30) at three of its
    own sizes, against the oracle word for word, and unpacked back."""
    n = 1 << k
    x = torch.randn(n, generator=gen(100 + k))
    x[:5] = torch.tensor([0.0, -0.0, float("nan"), float("inf"), -float("inf")])
    xd = x.to(DEV)
    got = ops.pack_sign(xd, mode)
    want = co.pack_sign_f32(x.numpy(), mode)
    assert np.array_equal(u64(got), want)
    bits = (x >= 0) if mode == 1 else (x > 0)
    assert torch.equal(ops.unpack_bool(got, [n]).cpu(), bits)
    assert int(ops.packed_popcount(got)) == int(bits.sum())
    pm1 = ops.unpack_bits(got, [n])
    assert torch.equal(pm1.cpu(), bits.float() * 2 - 1)


def test_ragged_bool_pair_full_chain(ops, co):
    """bool [4096, 4097], Bernoulli(0.3) (65 words per row, one valid bit in the last): pack, unpack,
    popcount-sum and AND / OR / XOR / NOT on the pair, every step against the oracle."""
    shape = (4096, 4097)
    a = torch.rand(shape, generator=gen(4097)) < 0.3
    b = torch.rand(shape, generator=gen(4098)) < 0.3
    pa, pb = ops.pack_bool(a.to(DEV)), ops.pack_bool(b.to(DEV))
    wa, wb = co.pack_bool(a.numpy()), co.pack_bool(b.numpy())
    assert tuple(pa.shape) == (4096, 65)
    assert np.array_equal(u64(pa), wa) and np.array_equal(u64(pb), wb)
    assert torch.equal(ops.unpack_bool(pa, list(shape)).cpu(), a)
    assert np.array_equal(ops.unpack_bits(pb, list(shape)).cpu().numpy(), co.unpack_pm1(wb, shape))
    assert int(ops.packed_popcount(pa)) == co.popcount_total(wa) == int(a.sum())
    assert int(ops.bit1_hamming_total(pa, pb)) == co.hamming_total(wa, wb) == int((a ^ b).sum())
    assert np.array_equal(ops.popcount(pa).cpu().numpy(), co.popcount_elems(wa.view(np.int64)))
    for code, name, ref in ((0, "and", a & b), (1, "or", a | b), (2, "xor", a ^ b), (3, "xnor", ~(a ^ b))):
        got = ops.bitwise_packed(pa, pb, code, 4097)
        assert np.array_equal(u64(got), co.bitwise(name, wa, wb, 4097)), name
        assert int(ops.packed_popcount(got)) == int(ref.sum()), name
    inv = ops.bit1_not_packed(pa, 4097)
    assert np.array_equal(u64(inv), co.bitwise("not", wa, None, 4097))
    assert int(ops.packed_popcount(inv)) == a.numel() - int(a.sum())
    # the same chain through the front end
    import brute_b200 as brute
    A, B = brute.Tensor(a.to(DEV), dtype=brute.bit1), brute.Tensor(b.to(DEV), dtype=brute.bit1)
    assert int(((A & B) | ~(A ^ B)).sum()) == int(((a & b) | ~(a ^ b)).sum())
    assert torch.equal((~A).bool().as_subclass(torch.Tensor).cpu(), ~a)


def test_known_answers(ops, golden):
    x = torch.from_numpy(golden["ka_float_in"]).to(DEV)
    got = ops.unpack_bool(ops.pack_sign(x, 0), [4]).cpu().numpy()
    assert np.array_equal(got, golden["ka_float_bits_gt0"])
    bits = torch.from_numpy(golden["ka_pm1_bits"]).to(DEV)
    assert np.array_equal(ops.unpack_bits(ops.pack_bool(bits), [5]).cpu().numpy(), golden["ka_pm1_out"])


# ---------------------------------------------------------------------------
# popcount / bitwise
# ---------------------------------------------------------------------------
def test_popcount_golden(ops, golden):
    for idx in range(int(golden["pop_count"])):
        packed = torch.from_numpy(golden[f"pop{idx}_packed"]).to(DEV)
        assert np.array_equal(ops.popcount(packed).cpu().numpy(), golden[f"pop{idx}_words"])
        assert int(ops.packed_popcount(packed)) == int(golden[f"pop{idx}_total"])
    assert np.array_equal(ops.popcount(torch.from_numpy(golden["pop_u8_in"]).to(DEV)).cpu().numpy(), golden["pop_u8_out"])
    assert np.array_equal(ops.popcount(torch.from_numpy(golden["pop_i32_in"]).to(DEV)).cpu().numpy(), golden["pop_i32_out"])


@pytest.mark.parametrize("dtype", [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64, torch.bool])
@pytest.mark.parametrize("n", [1, 15, 16, 17, 1000, 65537])
def test_popcount_elems_dtypes(ops, co, dtype, n):
    if dtype == torch.bool:
        x = torch.rand(n, generator=gen(n)) < 0.5
    else:
        info = torch.iinfo(dtype)
        x = torch.randint(info.min, info.max, (n,), generator=gen(n), dtype=torch.int64).to(dtype)
    got = ops.popcount(x.to(DEV))
    assert got.dtype == torch.int32
    assert np.array_equal(got.cpu().numpy(), co.popcount_elems(x.numpy()))
    # a view that is not 16-byte aligned takes the element-wise path
    if n > 3:
        assert np.array_equal(ops.popcount(x.to(DEV)[1:]).cpu().numpy(), co.popcount_elems(x[1:].numpy()))
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        ops.popcount(torch.zeros(4, device=DEV))


def test_totals_many_launches_in_flight_on_two_streams(ops, co):
    """The totals run as one launch each: blocks add into an accumulator in static device memory that the
    last block hands over and leaves zero. 700 launches queued without a sync, on two streams, walk the
    ring of accumulators almost three times; every result must still be its own input's count."""
    sizes = [1, 77, 4096, 100003, 1 << 18]
    hosts = [torch.randint(-2 ** 63, 2 ** 63 - 1, (n,), generator=gen(900 + i), dtype=torch.int64) for i, n in enumerate(sizes)]
    devs = [h.to(DEV) for h in hosts]
    want_pop = [co.popcount_total(h.numpy()) for h in hosts]
    want_ham = [co.hamming_total(hosts[i].numpy(), hosts[i].flip(0).contiguous().numpy()) for i in range(len(hosts))]
    flipped = [d.flip(0).contiguous() for d in devs]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = []
    for k in range(700):
        i = k % len(sizes)
        with torch.cuda.stream(streams[k & 1]):
            if k % 3 == 0:
                got.append((ops.bit1_hamming_total(devs[i], flipped[i]), want_ham[i]))
            else:
                got.append((ops.packed_popcount(devs[i]), want_pop[i]))
    torch.cuda.synchronize()
    bad = [(k, int(t), w) for k, (t, w) in enumerate(got) if int(t) != w]
    assert not bad, bad[:5]


@pytest.mark.parametrize("n_words", [0, 1, 2, 3, 255, 256, 257, 100003, 1 << 20])
def test_totals(ops, co, n_words):
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (n_words,), generator=gen(n_words), dtype=torch.int64)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (n_words,), generator=gen(n_words + 1), dtype=torch.int64)
    da, db = a.to(DEV), b.to(DEV)
    assert int(ops.packed_popcount(da)) == co.popcount_total(a.numpy())
    assert int(ops.bit1_hamming_total(da, db)) == co.hamming_total(a.numpy(), b.numpy())
    assert np.array_equal(ops.hamming_distance(da, db).cpu().numpy(), co.hamming_words(a.numpy(), b.numpy()))
    if n_words > 4:   # misaligned views, equal and different misalignment
        assert int(ops.packed_popcount(da[1:])) == co.popcount_total(a[1:].numpy())
        assert int(ops.bit1_hamming_total(da[1:], db[1:])) == co.hamming_total(a[1:].numpy(), b[1:].numpy())
        assert int(ops.bit1_hamming_total(da[1:-1], db[2:])) == co.hamming_total(a[1:-1].numpy(), b[2:].numpy())
    # byte-typed buffers with a tail that is not a whole word
    if n_words > 2:
        u = a.view(torch.uint8)[: n_words * 8 - 3].contiguous()
        assert int(ops.packed_popcount(u.to(DEV))) == co.popcount_total(u.numpy())
    with pytest.raises(RuntimeError, match="shape mismatch"):
        ops.bit1_hamming_total(da, torch.zeros(n_words + 1, dtype=torch.int64, device=DEV))


@pytest.mark.parametrize("shape", [(1,), (7,), (64,), (65,), (3, 13), (4, 64), (7, 130), (33, 1003), (4096, 4097 // 8),
                                   (1000, 7), (2, 3, 65)])
def test_bitwise_family(ops, co, shape):
    n = shape[-1]
    x = torch.rand(shape, generator=gen(n)) < 0.3
    y = torch.rand(shape, generator=gen(n + 1)) < 0.5
    c = torch.rand(shape, generator=gen(n + 2)) < 0.5
    px, py, pc = ops.pack_bool(x.to(DEV)), ops.pack_bool(y.to(DEV)), ops.pack_bool(c.to(DEV))
    for code, name in enumerate(["and", "or", "xor", "xnor", "andnot"]):
        got = ops.bitwise_packed(px, py, code, n)
        assert np.array_equal(u64(got), co.bitwise(name, u64(px), u64(py), n)), name
    inv = ops.bit1_not_packed(px, n)
    assert np.array_equal(u64(inv), co.bitwise("not", u64(px), None, n))
    assert int(ops.packed_popcount(inv)) == x.numel() - int(x.sum())
    assert np.array_equal(u64(ops.select_packed(pc, px, py)), co.select(u64(pc), u64(px), u64(py)))
    assert np.array_equal(ops.row_any(px).cpu().numpy(), x.any(dim=-1).numpy())
    assert np.array_equal(ops.row_all(px, n).cpu().numpy(), x.all(dim=-1).numpy())
    ones = ops.bitwise_packed(px, inv, 1, n)
    assert bool(ops.row_all(ones, n).all())


def test_not_pad_safe_sizes(ops, golden):
    for n in golden["ka_not_sizes"]:
        n = int(n)
        src = torch.rand(n, generator=gen(n)) < 0.5
        p = ops.pack_bool(src.to(DEV))
        inv = ops.bit1_not_packed(p, n)
        assert int(ops.packed_popcount(inv)) == n - int(src.sum())
        assert torch.equal(ops.unpack_bool(inv, [n]).cpu(), ~src)


# ---------------------------------------------------------------------------
# GEMM
# ---------------------------------------------------------------------------
def impls():
    from brute_b200 import _lib as L
    return {"auto": L.GEMM_AUTO, "popc": L.GEMM_POPC, "mma_b1": L.GEMM_MMA_B1, "tcgen05": L.GEMM_TCGEN05}


def status_ok():
    from brute_b200 import _lib as L
    return L.load().brute_b200_device_status() == 0


@pytest.mark.parametrize("M,N,K", [(64, 512, 4096), (128, 4096, 16384), (1, 256, 8192), (200, 300, 6400), (130, 700, 2048 + 128)])
def test_gemm_split_k(ops, co, M, N, K):
    # few tiles, long K: the one-CTA kernel splits K over blockIdx.z and the parts add up in the
    # zeroed output (integer adds: still bit-exact). Through the C ABI with ldc > N, so that the
    # columns past N must keep their sentinel (only the [M, N] block may be zeroed and written).
    from brute_b200 import _lib as L
    g = gen(M + N)
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (M, K // 64), generator=g, dtype=torch.int64)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (N, K // 64), generator=g, dtype=torch.int64)
    want = co.xnor_gemm(u64(a), u64(b), K)
    ad, bd = a.to(DEV), b.to(DEV)
    assert np.array_equal(ops.xnor_popcount_matmul(ad, bd, K).cpu().numpy(), want)
    ldc = N + 12
    c = torch.full((M, ldc), 7777, dtype=torch.int32, device=DEV)
    rc = L.load().brute_b200_xnor_gemm(ad.data_ptr(), bd.data_ptr(), c.data_ptr(), M, N, K // 64, K, ldc,
                                       L.GEMM_TCGEN05, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = c.cpu().numpy()
    assert np.array_equal(got[:, :N], want) and (got[:, N:] == 7777).all()
    for _ in range(20):                       # repeated launches into the same buffer
        ops.xnor_popcount_matmul(ad, bd, K)
    assert np.array_equal(ops.xnor_popcount_matmul(ad, bd, K).cpu().numpy(), want)
    assert status_ok()


def test_gemm_golden(ops, golden):
    for idx, (M, K, N) in enumerate(golden["gemm_cases"]):
        ap = torch.from_numpy(golden[f"gemm{idx}_ap"]).to(DEV)
        bp = torch.from_numpy(golden[f"gemm{idx}_bp"]).to(DEV)
        for name, impl in impls().items():
            Kp = ap.shape[1]
            if name in ("mma_b1", "tcgen05") and Kp % 2:
                with pytest.raises(RuntimeError):
                    ops.xnor_popcount_matmul_impl(ap, bp, int(K), impl)
                continue
            got = ops.xnor_popcount_matmul_impl(ap, bp, int(K), impl)
            assert got.dtype == torch.int32
            assert np.array_equal(got.cpu().numpy(), golden[f"gemm{idx}_c"]), (name, M, K, N)
    assert status_ok()


GEMM_SHAPES = [(1, 128, 1), (5, 128, 7), (128, 128, 256), (130, 256, 258), (127, 1024, 255), (256, 2048, 512),
               (300, 640, 700), (64, 8192, 64), (1, 4096, 1000), (513, 384, 129)]


@pytest.mark.parametrize("impl_name", ["popc", "mma_b1", "tcgen05", "auto"])
@pytest.mark.parametrize("M,K,N", GEMM_SHAPES)
def test_gemm_vs_oracle(ops, co, impl_name, M, K, N):
    a = torch.randint(0, 2, (M, K), generator=gen(M + K)).bool()
    b = torch.randint(0, 2, (N, K), generator=gen(N + K + 1)).bool()
    ap, bp = ops.pack_bool(a.to(DEV)), ops.pack_bool(b.to(DEV))
    want = co.xnor_gemm(u64(ap), u64(bp), K)
    got = ops.xnor_popcount_matmul_impl(ap, bp, K, impls()[impl_name]).cpu().numpy()
    assert np.array_equal(got, want)
    assert status_ok()


PAIR_SHAPES = [(129, 128, 1), (130, 256, 258), (256, 2048, 512), (300, 640, 700), (513, 384, 129),
               (257, 128 * 13, 255), (1024, 4096, 1024), (384, 128 * 25, 300), (2048, 128, 2048),
               (2048, 384, 4096), (1500, 1152, 5003), (4100, 256, 2052)]   # more tiles than SM pairs


@pytest.mark.parametrize("M,K,N", PAIR_SHAPES)
def test_gemm_pair_vs_oracle(ops, co, M, K, N):
    # two CTAs (cta_group::2) per 256 x 256 tile: ragged M and N, K-block counts that leave the
    # 12-step unroll and the 4-block packed stage at every remainder
    from brute_b200 import _lib as L
    a = torch.randint(0, 2, (M, K), generator=gen(M + K)).bool()
    b = torch.randint(0, 2, (N, K), generator=gen(N + K + 1)).bool()
    ap, bp = ops.pack_bool(a.to(DEV)), ops.pack_bool(b.to(DEV))
    want = co.xnor_gemm(u64(ap), u64(bp), K)
    for _ in range(2):      # twice: the second launch meets the first one's tensor-memory release
        got = ops.xnor_popcount_matmul_impl(ap, bp, K, L.GEMM_TCGEN05_PAIR).cpu().numpy()
        assert np.array_equal(got, want)
    assert status_ok()


def test_host_matmul_overlapped(ops, co):
    # host operands and result, blocks of rows on three streams; ragged last block
    import brute_b200 as brute
    M, K, N = 1000, 1024, 700
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (M, K // 64), generator=gen(5), dtype=torch.int64).pin_memory()
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (N, K // 64), generator=gen(6), dtype=torch.int64).pin_memory()
    want = co.xnor_gemm(a.numpy(), b.numpy(), K)
    out = torch.full((M, N), -1, dtype=torch.int32).pin_memory()
    for rows in (2048, 300, 128):
        out.fill_(-1)
        got = brute.host_matmul(a, b, K, out=out, rows_per_block=rows)
        torch.cuda.synchronize()
        assert got is out and np.array_equal(out.numpy(), want), rows
    fresh = brute.host_matmul(a, b, K)
    torch.cuda.synchronize()
    assert fresh.is_pinned() and np.array_equal(fresh.numpy(), want)
    with pytest.raises(RuntimeError, match="out must be"):
        brute.host_matmul(a, b, K, out=torch.empty((M, N + 1), dtype=torch.int32))


def test_gemm_pair_needs_two_row_blocks(ops):
    from brute_b200 import _lib as L
    a = torch.zeros((128, 2), dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError):
        ops.xnor_popcount_matmul_impl(a, a, 128, L.GEMM_TCGEN05_PAIR)


@pytest.mark.parametrize("M,K,N", [(3, 13, 5), (9, 100, 12), (33, 257, 66), (8, 65, 8), (32, 1, 32), (40, 777, 50)])
def test_gemm_k_not_multiple_of_64(ops, co, M, K, N):
    # K tails, as the reference fuzzes them (tests/fuzz/test_fuzz_matmul.py:15-34); odd word
    # counts are only accepted by the CUDA-core path, which AUTO then picks
    a = torch.randint(0, 2, (M, K), generator=gen(K)).bool()
    b = torch.randint(0, 2, (N, K), generator=gen(K + 1)).bool()
    ap, bp = ops.pack_bool(a.to(DEV)), ops.pack_bool(b.to(DEV))
    got = ops.xnor_popcount_matmul(ap, bp, K).cpu().numpy()
    ref = (a.float() * 2 - 1) @ (b.float() * 2 - 1).t()
    assert np.array_equal(got, ref.numpy().astype(np.int32))
    assert np.array_equal(got, co.xnor_gemm(u64(ap), u64(bp), K))


def test_gemm_errors_and_empty(ops):
    a = torch.zeros((4, 2), dtype=torch.int64, device=DEV)
    with pytest.raises(RuntimeError, match="must be 2-D"):
        ops.xnor_popcount_matmul(a[0], a, 128)
    with pytest.raises(RuntimeError, match="packed K mismatch"):
        ops.xnor_popcount_matmul(a, torch.zeros((4, 3), dtype=torch.int64, device=DEV), 128)
    assert tuple(ops.xnor_popcount_matmul(a[:0], a, 128).shape) == (0, 4)
    assert tuple(ops.xnor_popcount_matmul(a, a[:0], 128).shape) == (4, 0)
    z = ops.xnor_popcount_matmul(torch.zeros((3, 0), dtype=torch.int64, device=DEV),
                                 torch.zeros((5, 0), dtype=torch.int64, device=DEV), 0)
    assert tuple(z.shape) == (3, 5) and int(z.abs().sum()) == 0


def test_gemm_config1_all_paths(ops, co):
    # BASELINE config 1: 1024 x 1024 x 4096, Bernoulli(0.5) bits
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (1024, 64), generator=gen(1234), dtype=torch.int64)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (1024, 64), generator=gen(1235), dtype=torch.int64)
    want = co.xnor_gemm(a.numpy(), b.numpy(), 4096)
    for name, impl in impls().items():
        got = ops.xnor_popcount_matmul_impl(a.to(DEV), b.to(DEV), 4096, impl).cpu().numpy()
        assert np.array_equal(got, want), name
    assert status_ok()


def test_gemm_large_properties(ops):
    # BASELINE config 3 scale (16384^3 is checked by structure, not against the CPU):
    #  * the tensor-core path equals the CUDA-core path bit for bit on a 4096-row slab,
    #  * a row of A against itself gives K on the diagonal, and -K against its complement.
    K = 16384
    Kp = K // 64
    g = gen(3)
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (16384, Kp), generator=g, dtype=torch.int64).to(DEV)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (16384, Kp), generator=g, dtype=torch.int64).to(DEV)
    c = ops.xnor_popcount_matmul(a, b, K)
    assert tuple(c.shape) == (16384, 16384)
    slab = ops.xnor_popcount_matmul_impl(a[:512], b[:4096], K, impls()["popc"])
    assert torch.equal(c[:512, :4096], slab)
    from brute_b200 import _lib as L
    for impl in (L.GEMM_TCGEN05, L.GEMM_TCGEN05_PAIR):
        assert torch.equal(ops.xnor_popcount_matmul_impl(a, b, K, impl), c)
    # linearity in the hamming domain: C(a, b) + C(a, ~b) == 0
    c2 = ops.xnor_popcount_matmul(a[:1024], torch.bitwise_not(b[:2048]), K)
    assert int((c[:1024, :2048] + c2).abs().max()) == 0
    d = ops.xnor_popcount_matmul(a[:2048], a[:2048], K)
    assert bool((d.diagonal() == K).all()) and bool((d == d.t()).all())
    assert int(c.abs().max()) <= K and int((c & 1).sum()) == 0
    assert status_ok()


@pytest.mark.parametrize("impl_name", ["tcgen05", "tcgen05_pair"])
def test_gemm_repeatable_under_load(ops, impl_name):
    # 8192 tiles per launch, 60 launches, every one compared with the CUDA-core kernel: the
    # pipelines hand shared-memory slots between TMA, expander warps and the tensor core, and a
    # slot released one instruction too early shows up as one wrong tile in about 10^5
    from brute_b200 import _lib as L
    K = 16384
    g = gen(11)
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (16384, K // 64), generator=g, dtype=torch.int64).to(DEV)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (16384, K // 64), generator=g, dtype=torch.int64).to(DEV)
    ref = ops.xnor_popcount_matmul_impl(a, b, K, L.GEMM_POPC)
    impl = {"tcgen05": L.GEMM_TCGEN05, "tcgen05_pair": L.GEMM_TCGEN05_PAIR}[impl_name]
    for it in range(60):
        c = ops.xnor_popcount_matmul_impl(a, b, K, impl)
        assert torch.equal(c, ref), f"launch {it}"
        del c
    assert status_ok()


@pytest.mark.parametrize("impl_name", ["popc", "mma_b1", "tcgen05", "tcgen05_pair"])
@pytest.mark.parametrize("mode", [0, 1])
def test_mlp_layer(ops, co, impl_name, mode):
    from brute_b200 import _lib as L
    M, K, N = 200, 512, 330
    a = torch.randint(0, 2, (M, K), generator=gen(1)).bool()
    w = torch.randint(0, 2, (N, K), generator=gen(2)).bool()
    scale = torch.rand(N, generator=gen(3)) + 0.5
    ap, wp = ops.pack_bool(a.to(DEV)), ops.pack_bool(w.to(DEV))
    want = co.xnor_gemm_scale_sign_pack(u64(ap), u64(wp), scale.numpy(), K, mode)
    out = torch.empty((M, (N + 63) // 64), dtype=torch.int64, device=DEV)
    rc = L.load().brute_b200_xnor_gemm_scale_sign_pack(
        ap.data_ptr(), wp.data_ptr(), scale.to(DEV).data_ptr(), out.data_ptr(), M, N, K // 64, K, mode,
        {**impls(), "tcgen05_pair": L.GEMM_TCGEN05_PAIR}[impl_name], torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert np.array_equal(u64(out), want)
    assert np.array_equal(u64(ops.xnor_matmul_scale_sign_pack(ap, wp, scale.to(DEV), K, mode)), want)


@pytest.mark.parametrize("impl_name", ["popc", "tcgen05", "tcgen05_pair"])
@pytest.mark.parametrize("mode", [0, 1])
def test_mlp_layer_special_scales(ops, co, impl_name, mode):
    # sign(scale * C) for every kind of scale: the pair kernel decides it in integers (a sign and an
    # offset per column), the others multiply; both must give what the float product gives, also where
    # C = 0 (0 * inf is NaN and compares false) and for zero, negative, denormal and NaN scales
    from brute_b200 import _lib as L
    M, K, N = 300, 256, 520
    a = torch.randint(0, 2, (M, K), generator=gen(21)).bool()
    w = torch.randint(0, 2, (N, K), generator=gen(22)).bool()
    w[:16] = a[:16]
    w[:16, : K // 2] ^= True                       # rows 0..15 of A against columns 0..15: C = 0
    specials = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1e-42, -1e-42, -2.5,
                             3.0e38, -3.0e38, 1.0, -1.0], dtype=torch.float32)
    scale = torch.rand(N, generator=gen(23)) - 0.5
    for i in range(N):
        if i % 3 != 2:
            scale[i] = specials[(i // 3 + i) % len(specials)]
    ap, wp = ops.pack_bool(a.to(DEV)), ops.pack_bool(w.to(DEV))
    c = co.xnor_gemm(u64(ap), u64(wp), K)
    assert (c[:16, :16].diagonal() == 0).all()
    want = co.xnor_gemm_scale_sign_pack(u64(ap), u64(wp), scale.numpy(), K, mode)
    out = torch.empty((M, (N + 63) // 64), dtype=torch.int64, device=DEV)
    rc = L.load().brute_b200_xnor_gemm_scale_sign_pack(
        ap.data_ptr(), wp.data_ptr(), scale.to(DEV).data_ptr(), out.data_ptr(), M, N, K // 64, K, mode,
        {**impls(), "tcgen05_pair": L.GEMM_TCGEN05_PAIR}[impl_name], torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert np.array_equal(u64(out), want)


def test_mlp_config4_chain(ops, co):
    # BASELINE config 4 at reduced batch against the oracle: 4096 -> 16384 -> 4096
    import brute_b200 as brute
    g = gen(4)
    x = torch.randn((256, 4096), generator=g)
    w1 = torch.randn((16384, 4096), generator=g)
    w2 = torch.randn((4096, 16384), generator=g)
    s1 = torch.rand(16384, generator=g) + 0.5
    s2 = torch.rand(4096, generator=g) + 0.5
    xb, w1b, w2b = (brute.pack_sign(t.to(DEV), ge0=True) for t in (x, w1, w2))
    h = brute.binary_linear(xb, w1b, s1.to(DEV))
    y = brute.binary_linear(h, w2b, s2.to(DEV))
    xp, w1p, w2p = (co.pack_sign_f32(t.numpy(), 1) for t in (x, w1, w2))
    hp = co.xnor_gemm_scale_sign_pack(xp, w1p, s1.numpy(), 4096, 1)
    yp = co.xnor_gemm_scale_sign_pack(hp, w2p, s2.numpy(), 16384, 1)
    assert np.array_equal(u64(h._packed_buf), hp)
    assert np.array_equal(u64(y._packed_buf), yp)


# ---------------------------------------------------------------------------
# layout: bit-matrix transpose, any/all over a non-packed axis
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 1), (3, 5), (64, 64), (65, 63), (130, 257), (256, 256), (257, 1000), (1000, 257),
                                   (2, 3, 70, 129), (5, 300, 64), (4096, 4097), (1, 100000), (100000, 1),
                                   # even word counts on both sides: the TMA kernel (ragged rows, ragged bits, batches)
                                   (640, 384), (1000, 8192), (2, 3, 128, 256), (1408, 896), (5107, 6395), (65, 100)])
def test_transpose_packed(ops, co, shape):
    import brute_b200 as brute
    x = torch.rand(shape, generator=gen(sum(shape))) < 0.5
    p = ops.pack_bool(x.to(DEV))
    got = ops.transpose_packed(p, shape[-2], shape[-1])
    assert tuple(got.shape) == shape[:-2] + (shape[-1], (shape[-2] + 63) // 64)
    assert np.array_equal(u64(got), co.pack_bool(x.transpose(-1, -2).contiguous().numpy()))
    assert np.array_equal(u64(got), co.transpose_bits(u64(p), shape[-2], shape[-1]))
    # involution, and the front end takes this path for .transpose(-1, -2) of a packed tensor
    assert torch.equal(ops.transpose_packed(got, shape[-1], shape[-2]), p)
    b = brute.Tensor(x.to(DEV), dtype=brute.bit1)
    bt = b.transpose(-1, -2)
    assert torch.equal(bt._packed_buf, got)
    assert torch.equal(bt.bool().as_subclass(torch.Tensor).cpu(), x.transpose(-1, -2))


@pytest.mark.parametrize("shape,dim", [((5, 70), 0), ((1, 3), 0), ((4, 6, 130), 1), ((4, 6, 130), 0), ((2, 1, 64), 1),
                                       ((1000, 4097), 0), ((3, 100000, 65), 1), ((70000, 64), 0),
                                       # rows of whole 16-byte vectors: the slab kernel, with and without a cluster split of the rows
                                       ((4096, 128), 0), ((5000, 8192), 0), ((3, 70, 256), 1), ((2, 1000, 128 * 70), 1),
                                       ((9, 20000), 0), ((33, 2, 64 * 6), 0), ((1, 128), 0), ((64, 64 * 66 - 3), 0)])
def test_reduce_rows_packed(ops, co, shape, dim):
    import brute_b200 as brute
    x = torch.rand(shape, generator=gen(sum(shape))) < 0.999
    x[..., 0] = False        # some all-false columns for any()
    p = ops.pack_bool(x.to(DEV))
    for use_or, ref in ((True, x.any(dim=dim)), (False, x.all(dim=dim))):
        got = ops.reduce_rows_packed(p, dim, use_or)
        assert np.array_equal(u64(got), co.pack_bool(ref.numpy())), use_or
    b = brute.Tensor(x.to(DEV), dtype=brute.bit1)
    assert torch.equal(b.any(dim=dim).bool().as_subclass(torch.Tensor).cpu(), x.any(dim=dim))
    assert torch.equal(b.all(dim=dim).bool().as_subclass(torch.Tensor).cpu(), x.all(dim=dim))
    with pytest.raises(RuntimeError, match="non-packed"):
        ops.reduce_rows_packed(p, len(shape) - 1, True)


@pytest.mark.parametrize("shape", [(1,), (5,), (64,), (65,), (3, 130), (2, 3, 257), (4, 1003), (7, 4097), (1, 1 << 20), (300, 6400),
                                   # even word counts >= 64 per row: the vector kernel (exact, ragged, partial last chunk)
                                   (3, 4096), (5, 4096 + 64), (4, 64 * 66 - 5), (2, 64 * 130 - 63), (9, 8192 + 128 - 1),
                                   (2, 3, 64 * 64 * 3), (1, (1 << 20) - 5), (17, 64 * 200),
                                   (3, 64 * 130 - 7), (2, 64 * 258 - 1), (5, 64 * 126), (2, 64 * 254 - 33)])
def test_flip_roll_gather_packed(ops, co, shape):
    x = torch.rand(shape, generator=gen(sum(shape))) < 0.5
    n = shape[-1]
    p = ops.pack_bool(x.to(DEV))
    assert np.array_equal(u64(ops.flip_packed(p, n)), co.pack_bool(torch.flip(x, [-1]).numpy()))
    for shift in (0, 1, -1, 63, 64, 65, n - 1, n, 3 * n + 7, -2 * n - 5, n // 2):
        assert np.array_equal(u64(ops.roll_packed(p, n, shift)), co.pack_bool(torch.roll(x, shift, -1).numpy())), shift
    idx = torch.randint(0, n, (min(2 * n + 3, 100000),), generator=gen(n))
    got = ops.gather_packed(p, idx.to(DEV), n)
    assert np.array_equal(u64(got), co.pack_bool(x.index_select(-1, idx).numpy()))
    assert np.array_equal(u64(got), co.gather_bits(u64(p), idx.numpy(), n))
    # an index outside the row reads as 0 at the C ABI (the front end raises before it gets there)
    bad = idx.clone()
    bad[0] = n
    assert np.array_equal(u64(ops.gather_packed(p, bad.to(DEV), n)), co.gather_bits(u64(p), bad.numpy(), n))


# ---------------------------------------------------------------------------
# signed_bundle
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("B,M,N,D", [(1, 1, 1, 1), (2, 5, 7, 70), (1, 33, 130, 128), (3, 64, 256, 64),
                                     (2, 100, 1000, 200), (1, 32, 128, 4096),
                                     # tensor-core path (N % 16 == 0, N >= 128, M >= 64): ragged M, N, D
                                     (2, 128, 256, 128), (1, 200, 1024, 70), (3, 64, 128, 200), (1, 1000, 2048, 128),
                                     (2, 130, 144, 64), (1, 257, 4096 + 16, 129), (4, 64, 128, 1)])
def test_signed_bundle(ops, co, B, M, N, D):
    import brute_b200 as brute
    g = gen(B + M + N + D)
    lo, hi = (-3, 4) if (B + M) % 2 else (-128, 128)        # small votes (many ties) or the full int8 range
    W = torch.randint(lo, hi, (B, M, N), generator=g, dtype=torch.int64).to(torch.int8)
    v = torch.rand((B, N, D), generator=g) < 0.5
    vp = ops.pack_bool(v.to(DEV))
    got = ops.signed_bundle(W.to(DEV), vp, D)
    assert np.array_equal(u64(got), co.signed_bundle(W.numpy(), u64(vp), D))
    for _ in range(5):          # same answer launch after launch (the tensor path pipelines TMA, expanders and MMAs)
        assert torch.equal(ops.signed_bundle(W.to(DEV), vp, D), got)
    # through the front-end helper, against the +-1 integer contraction
    out = brute.fast.signed_bundle(W.to(DEV), brute.Tensor(v.to(DEV), dtype=brute.bit1))
    acc = torch.einsum("bmn,bnd->bmd", W.float(), v.float() * 2 - 1)
    assert out.dtype == brute.bit1 and torch.equal(out.bool().as_subclass(torch.Tensor).cpu(), acc >= 0)
    with pytest.raises(RuntimeError, match="must be int8"):
        ops.signed_bundle(W.to(DEV).int(), vp, D)


def test_signed_bundle_workspace_contract(ops, co):
    # the C entry point allocates nothing: without enough scratch it refuses, and says so
    from brute_b200 import _lib as L
    lib = L.load()
    B, M, N, D = 2, 128, 256, 128
    g = gen(9)
    W = torch.randint(-5, 6, (B, M, N), generator=g, dtype=torch.int64).to(torch.int8).to(DEV)
    vp = ops.pack_bool((torch.rand((B, N, D), generator=g) < 0.5).to(DEV))
    out = torch.zeros((B, M, 2), dtype=torch.int64, device=DEV)
    need = int(lib.brute_b200_signed_bundle_workspace_bytes(B, N, D))
    assert need == B * D * (N // 64) * 8
    ws = torch.empty(need // 8, dtype=torch.int64, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    args = (W.data_ptr(), vp.data_ptr(), out.data_ptr(), B, M, N, 2, D)
    assert lib.brute_b200_signed_bundle_ws(*args, None, 0, st) == L.ERR_WORKSPACE
    assert lib.brute_b200_signed_bundle_ws(*args, ws.data_ptr(), need - 8, st) == L.ERR_WORKSPACE
    assert "scratch" in L.strerror(L.ERR_WORKSPACE)
    assert lib.brute_b200_signed_bundle_ws(*args, ws.data_ptr(), need, st) == 0
    assert np.array_equal(u64(out), co.signed_bundle(W.cpu().numpy(), u64(vp), D))
    # a shape outside the tensor path needs no workspace at all
    W2 = W[:, :, :100].contiguous()
    v2 = vp[:, :100].contiguous()
    assert lib.brute_b200_signed_bundle_ws(W2.data_ptr(), v2.data_ptr(), out.data_ptr(), B, M, 100, 2, D, None, 0, st) == 0
    assert np.array_equal(u64(out), co.signed_bundle(W2.cpu().numpy(), u64(v2), D))
    assert status_ok()


# ---------------------------------------------------------------------------
# attention (parity unpinned: no reference kernel; oracle = composition)
# ---------------------------------------------------------------------------
ATT_TOL = 2e-2      # relative to the largest |output|, the tolerance the task states for bf16


@pytest.mark.parametrize("B,H,S,D,causal", [(1, 2, 256, 128, True), (1, 1, 200, 128, True), (2, 2, 128, 64, True),
                                            (1, 2, 333, 128, False), (1, 1, 64, 64, False), (1, 1, 1, 128, True),
                                            (1, 3, 1000, 128, True), (1, 2, 1000, 64, True), (1, 2, 777, 64, False)])
def test_attention_vs_oracle(ops, co, B, H, S, D, causal):
    import brute_b200 as brute
    g = gen(S + D)
    q = torch.randn((B, H, S, D), generator=g)
    k = torch.randn((B, H, S, D), generator=g)
    v = torch.randn((B, H, S, D), generator=g).to(torch.bfloat16)
    qb, kb = brute.pack_sign(q.to(DEV), ge0=True), brute.pack_sign(k.to(DEV), ge0=True)
    out = brute.binary_attention(qb, kb, v.to(DEV), causal=causal)
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (B, H, S, D)
    want = co.binary_attention(co.pack_sign_f32(q.numpy(), 1), co.pack_sign_f32(k.numpy(), 1),
                               v.float().numpy(), causal, D ** -0.5)
    got = out.float().cpu().numpy()
    assert np.isfinite(got).all()
    mx, row = att_errors(got, want)
    assert mx <= ATT_TOL and row <= ATT_TOL, (mx, row)


def att_errors(got: np.ndarray, want: np.ndarray):
    """(max-norm error relative to the largest |output|, worst per-row relative L2 error)."""
    mx = float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-6))
    num = np.sqrt(((got - want) ** 2).sum(-1))
    den = np.maximum(np.sqrt((want ** 2).sum(-1)), 1e-6)
    return mx, float((num / den).max())


@pytest.mark.parametrize("D,H", [(128, 2), (64, 2)])
def test_attention_vs_oracle_at_full_sequence_length(ops, co, D, H):
    """S = 4096, causal: the benchmark configuration's sequence length on two heads, against the oracle,
    by the max norm and row by row (every query row's output vector within 2e-2 of the oracle's in
    relative L2 norm)."""
    import brute_b200 as brute
    S = 4096
    g = gen(4096 + D)
    q = torch.randn((1, H, S, D), generator=g)
    k = torch.randn((1, H, S, D), generator=g)
    v = torch.randn((1, H, S, D), generator=g).to(torch.bfloat16)
    qb, kb = brute.pack_sign(q.to(DEV), ge0=True), brute.pack_sign(k.to(DEV), ge0=True)
    got = brute.binary_attention(qb, kb, v.to(DEV), causal=True).float().cpu().numpy()
    want = co.binary_attention(co.pack_sign_f32(q.numpy(), 1), co.pack_sign_f32(k.numpy(), 1),
                               v.float().numpy(), True, D ** -0.5)
    mx, row = att_errors(got, want)
    print(f"attention S={S} D={D}: max-norm error {mx:.2e}, worst row-wise relative error {row:.2e} (limit {ATT_TOL})")
    assert np.isfinite(got).all()
    assert mx <= ATT_TOL and row <= ATT_TOL
    assert status_ok()


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("S,causal,scale", [(2048, True, None), (1111, False, None), (640, True, -0.05), (512, True, 0.5)])
def test_attention_kernels_agree(ops, co, monkeypatch, S, causal, scale, D):
    # each head dim has three kernels (tcgen05, mma.sync scores, CUDA-core scores) that round the weights
    # to bf16 the same way and differ only in the order of fp32 sums; scale 0.5 is too steep for the
    # table and takes the online-softmax kernel whatever the setting
    import brute_b200 as brute
    g = gen(S)
    q = torch.randn((1, 4, S, D), generator=g)
    k = torch.randn((1, 4, S, D), generator=g)
    v = torch.randn((1, 4, S, D), generator=g).to(torch.bfloat16).to(DEV)
    qb, kb = brute.pack_sign(q.to(DEV), ge0=True), brute.pack_sign(k.to(DEV), ge0=True)
    outs = {}
    for impl in ("tcgen05", "mma", "popc"):
        monkeypatch.setenv("BRUTE_ATTENTION_IMPL", impl)
        outs[impl] = brute.binary_attention(qb, kb, v, causal=causal, scale=scale).float()
    monkeypatch.delenv("BRUTE_ATTENTION_IMPL")
    ref = outs["popc"]
    for impl in ("tcgen05", "mma"):
        assert float((outs[impl] - ref).abs().max()) <= 1e-2 * float(ref.abs().max()), impl
    want = co.binary_attention(co.pack_sign_f32(q.numpy(), 1), co.pack_sign_f32(k.numpy(), 1),
                               v.float().cpu().numpy(), causal, D ** -0.5 if scale is None else scale)
    assert np.abs(outs["tcgen05"].cpu().numpy() - want).max() <= ATT_TOL * np.abs(want).max()
    assert status_ok()


@pytest.mark.parametrize("B,D", [(8, 128), (1, 128), (2, 64)])
def test_attention_repeatable_under_load(ops, B, D):
    # no atomics anywhere in the kernel: 30 launches of BASELINE config 5 must agree bit for bit
    # (a buffer handed over too early in the TMEM / shared-memory pipeline would show up here).
    # B = 8: tiles ordered head by head; B = 1 (one rank's share on 8 GPUs): all heads' K and V
    # fit in L2 and the tiles are ordered heavy-first across the heads; D = 64: the other instance.
    import brute_b200 as brute
    g = gen(8)
    q = brute.pack_sign(torch.randn((B, 32, 4096, D), generator=g).to(DEV), ge0=True)
    k = brute.pack_sign(torch.randn((B, 32, 4096, D), generator=g).to(DEV), ge0=True)
    v = torch.randn((B, 32, 4096, D), generator=g).to(torch.bfloat16).to(DEV)
    ref = brute.binary_attention(q, k, v, causal=True)
    for it in range(30):
        assert torch.equal(brute.binary_attention(q, k, v, causal=True), ref), f"launch {it}"
    assert status_ok()


def test_attention_first_row_is_v0(ops):
    # causal: query 0 sees only key 0, so the output row is exactly V[0]
    import brute_b200 as brute
    g = gen(5)
    q = torch.randn((2, 4, 512, 128), generator=g)
    k = torch.randn((2, 4, 512, 128), generator=g)
    v = torch.randn((2, 4, 512, 128), generator=g).to(torch.bfloat16).to(DEV)
    out = brute.binary_attention(brute.pack_sign(q.to(DEV)), brute.pack_sign(k.to(DEV)), v, causal=True)
    assert torch.equal(out[:, :, 0], v[:, :, 0])


def test_attention_config5_properties(ops):
    # BASELINE config 5 shape on one (b) slice of the full head count: constant V rows
    # must come back unchanged (softmax weights sum to 1), whatever the scores are.
    import brute_b200 as brute
    g = gen(6)
    B, H, S, D = 1, 32, 4096, 128
    q = torch.randn((B, H, S, D), generator=g)
    k = torch.randn((B, H, S, D), generator=g)
    row = torch.randn((B, H, 1, D), generator=g).to(torch.bfloat16)
    v = row.expand(B, H, S, D).contiguous().to(DEV)
    out = brute.binary_attention(brute.pack_sign(q.to(DEV), ge0=True), brute.pack_sign(k.to(DEV), ge0=True), v, causal=True)
    err = (out.float() - v.float()).abs().max() / v.float().abs().max()
    assert float(err) < ATT_TOL


# ---------------------------------------------------------------------------
# the bounded in-kernel wait: make one run out, on purpose and safely
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("relaxed", [0, 1])
def test_bounded_wait_gives_up_and_the_library_recovers(ops, co, relaxed):
    """Every tcgen05 kernel waits on mbarriers with a time limit; a wait that runs out records a code
    in a device status word, raises the CTA's abort flag and the kernel returns. Here a one-CTA test
    kernel waits 200 microseconds on a barrier that nothing arrives at: it must return, the status
    must read BRUTE_ERR_DEVICE_WAIT exactly once, and the next GEMM must be correct."""
    from brute_b200 import _lib as L
    lib = L.load()
    assert lib.brute_b200_device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.brute_b200_selftest_bounded_wait(200, relaxed, flag.data_ptr(), st) == 0
    torch.cuda.synchronize()                      # returns: the kernel ended by itself
    assert int(flag) == 3, "the waiter must see the timeout and the other warp the abort flag"
    assert lib.brute_b200_device_status() == L.ERR_DEVICE_WAIT
    assert lib.brute_b200_device_status() == 0, "reading the status clears it"
    assert lib.brute_b200_selftest_bounded_wait(0, relaxed, flag.data_ptr(), st) == L.ERR_INVALID_ARG
    # the library is usable afterwards: a tensor-core GEMM against the oracle
    M, N, K = 256, 512, 2048
    a = torch.rand((M, K), generator=gen(77)) < 0.5
    b = torch.rand((N, K), generator=gen(78)) < 0.5
    got = ops.xnor_popcount_matmul(ops.pack_bool(a.to(DEV)), ops.pack_bool(b.to(DEV)), K)
    assert np.array_equal(got.cpu().numpy(), co.xnor_gemm(co.pack_bool(a.numpy()), co.pack_bool(b.numpy()), K))
    assert status_ok()


# ---------------------------------------------------------------------------
# scatter along the packed axis
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("rows,n,n_idx", [(1, 64, 1), (7, 131, 40), (33, 1003, 1003), (4096, 4097, 512), (3, 200, 0),
                                          (70000, 65, 9)])
def test_scatter_bits_vs_oracle(ops, co, rows, n, n_idx):
    g = gen(rows + n + n_idx)
    x = torch.rand((rows, n), generator=g) < 0.5
    packed = ops.pack_bool(x.to(DEV))
    idx = torch.randperm(n, generator=g)[:n_idx]                   # distinct positions: the result is unique
    src = torch.rand((rows, n_idx), generator=g) < 0.5
    want_base = co.pack_bool(x.numpy())
    for value in (0, 1):
        got = ops.scatter_packed_(packed.clone(), idx.to(DEV), None, bool(value), n)
        assert np.array_equal(u64(got), co.scatter_bits(want_base, idx.numpy(), None, value, n)), value
    if n_idx:
        sp = ops.pack_bool(src.to(DEV))
        got = ops.scatter_packed_(packed.clone(), idx.to(DEV), sp, False, n)
        want = co.scatter_bits(want_base, idx.numpy(), co.pack_bool(src.numpy()), 0, n)
        assert np.array_equal(u64(got), want)
        ref = x.clone()
        ref[:, idx] = src
        assert np.array_equal(want, co.pack_bool(ref.numpy())), "oracle vs torch.bool"
    # repeated positions with one constant value are well defined; out-of-range positions write nothing
    rep = torch.tensor([0, n - 1, 0, n - 1, n + 5, -1], dtype=torch.int64)
    got = ops.scatter_packed_(packed.clone(), rep.to(DEV), None, True, n)
    assert np.array_equal(u64(got), co.scatter_bits(want_base, rep.numpy(), None, 1, n))


# ---------------------------------------------------------------------------
# transport of GEMM blocks between ranks (int16 on the wire, widened and laid out on arrival)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("world,rows,n_loc", [(2, 64, 128), (8, 33, 8), (3, 5, 7), (4, 1, 1000), (1, 17, 24)])
def test_narrow_and_unstack_rank_blocks(ops, world, rows, n_loc):
    g = gen(world * rows + n_loc)
    c = torch.randint(-32767, 32768, (world, rows, n_loc), generator=g, dtype=torch.int32)
    c[0, 0, 0], c[-1, -1, -1] = -32767, 32767
    cd = c.to(DEV)
    n16 = ops.narrow_i32_i16(cd)
    assert n16.dtype == torch.int16 and torch.equal(n16.cpu(), c.to(torch.int16))
    assert torch.equal(ops.narrow_i32_i16(cd.view(-1)[1:]).cpu(), c.view(-1)[1:].to(torch.int16))   # unaligned base
    want = c.permute(1, 0, 2).reshape(rows, world * n_loc)
    M = rows + 3
    for stacked in (n16, cd):
        out = torch.full((M, world * n_loc), 12345, dtype=torch.int32, device=DEV)
        ops.unstack_rank_blocks(stacked, out, 2)
        assert torch.equal(out[2:2 + rows].cpu(), want)
        assert bool((out[:2] == 12345).all()) and bool((out[2 + rows:] == 12345).all())


def _peer_tables(bufs, flags):
    import ctypes as C
    arr = C.c_void_p * len(bufs)
    return arr(*[b.data_ptr() for b in bufs]), arr(*[f.data_ptr() for f in flags])


@pytest.mark.parametrize("eb", [2, 4])
@pytest.mark.parametrize("world,M,n_loc,m0,m1", [(1, 40, 64, 0, 40), (2, 300, 2048, 0, 300), (4, 129, 136, 7, 120), (8, 2100, 512, 100, 2100)])
def test_gather_peer_widen_on_one_device(world, M, n_loc, m0, m1, eb):
    """The peer-memory exchange kernels with every "rank" played by a buffer of this one device: blocks of
    int16 (or, for K > 32767, int32) [M, n_loc] per rank, flags raised through the library, then rank
    `self`'s replicated int32 result must hold every rank's rows [m0, m1) in its column block and nothing else."""
    from brute_b200 import _lib as L
    lib = L.load()
    g = gen(world * M + n_loc)
    if eb == 2:
        blocks = [torch.randint(-32767, 32768, (M, n_loc), generator=g, dtype=torch.int16) for _ in range(world)]
    else:
        blocks = [torch.randint(-(1 << 30), 1 << 30, (M, n_loc), generator=g, dtype=torch.int32) for _ in range(world)]
    bufs = [b.to(DEV) for b in blocks]
    flags = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(world)]
    send, flg = _peer_tables(bufs, flags)
    stream = torch.cuda.current_stream().cuda_stream
    for p in range(world):
        L.check(lib.brute_b200_peer_set_flag(flags[p].data_ptr() + 4 * 3, 9, stream), "peer_set_flag")
    torch.cuda.synchronize()
    assert all(int(f[3]) == 9 for f in flags)
    want = torch.cat(blocks, dim=1).to(torch.int32)
    for self_rank in {0, world - 1}:
        for ctas in (1, 5):
            out = torch.full((M, world * n_loc), 777, dtype=torch.int32, device=DEV)
            L.check(lib.brute_b200_gather_peer_widen(send, flg, out.data_ptr(), M, n_loc, eb, m0, m1, world, self_rank,
                                                     3, 9, ctas, 2_000_000, stream), "gather_peer_widen")
            assert lib.brute_b200_peer_wait_status() == 0
            got = out.cpu()
            assert torch.equal(got[m0:m1], want[m0:m1])
            assert bool((got[:m0] == 777).all()) and bool((got[m1:] == 777).all())
    # waiting for an older call number is satisfied by a newer one (flags only grow)
    L.check(lib.brute_b200_peer_wait_flags(send, flg, world, 0, 3, 8, 2_000_000, stream), "peer_wait_flags")
    assert lib.brute_b200_peer_wait_status() == 0


def test_peer_wait_gives_up_and_reports_the_rank():
    """A flag that nobody raises: the bounded waits of the peer kernels run out after their limit (3 ms
    here), the kernels return, the status names the rank, and the next exchange works. Nothing hangs."""
    from brute_b200 import _lib as L
    lib = L.load()
    world, M, n_loc = 2, 64, 64
    bufs = [torch.ones((M, n_loc), dtype=torch.int16, device=DEV) * (p + 1) for p in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(world)]
    send, flg = _peer_tables(bufs, flags)
    stream = torch.cuda.current_stream().cuda_stream
    out = torch.zeros((M, world * n_loc), dtype=torch.int32, device=DEV)
    L.check(lib.brute_b200_gather_peer_widen(send, flg, out.data_ptr(), M, n_loc, 2, 0, M, world, 0, 5, 1, 2, 3000, stream), "gather")
    assert lib.brute_b200_peer_wait_status() == 1 + 1           # rank 1's flag did not arrive
    assert bool((out[:, :n_loc] == 1).all()) and bool((out[:, n_loc:] == 0).all())   # the own block needs no flag
    L.check(lib.brute_b200_peer_wait_flags(send, flg, world, 0, 5, 1, 3000, stream), "wait_flags")
    assert lib.brute_b200_peer_wait_status() == 1 + 1
    assert lib.brute_b200_peer_wait_status() == 0               # reading cleared it
    L.check(lib.brute_b200_peer_set_flag(flags[1].data_ptr() + 4 * 5, 1, stream), "set_flag")
    L.check(lib.brute_b200_gather_peer_widen(send, flg, out.data_ptr(), M, n_loc, 2, 0, M, world, 0, 5, 1, 2, 3000, stream), "gather")
    assert lib.brute_b200_peer_wait_status() == 0
    assert bool((out[:, n_loc:] == 2).all())


@pytest.mark.parametrize("M,K,N", [(512, 1024, 512), (300, 640, 700), (513, 384, 129), (1024, 16384, 2048), (2048, 32704, 256)])
def test_gemm_int16_output_equals_the_narrowed_int32_result(ops, M, K, N):
    """The GEMM variant that writes C as int16 from its epilogue (the transport form of a sharded result):
    equal to the int32 GEMM narrowed, into a wider destination (ldc > N) whose other columns stay put."""
    from brute_b200 import _lib as L
    lib = L.load()
    kp = (K + 63) // 64
    a = torch.randint(-2 ** 63, 2 ** 63 - 1, (M, kp), generator=gen(M + K), dtype=torch.int64).to(DEV)
    b = torch.randint(-2 ** 63, 2 ** 63 - 1, (N, kp), generator=gen(N + K), dtype=torch.int64).to(DEV)
    if K % 64:
        a[:, -1] &= (1 << (K % 64)) - 1
        b[:, -1] &= (1 << (K % 64)) - 1
    want = ops.xnor_popcount_matmul(a, b, K).to(torch.int16)
    ldc = N + 8
    for leave in (0, 32):
        out = torch.full((M, ldc), -7, dtype=torch.int16, device=DEV)
        rc = lib.brute_b200_xnor_gemm_i16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, kp, K, ldc, leave,
                                          torch.cuda.current_stream().cuda_stream)
        if rc == L.UNSUPPORTED:
            pytest.skip("shape outside the pair kernel")
        L.check(rc, "xnor_gemm_i16")
        assert torch.equal(out[:, :N], want)
        assert bool((out[:, N:] == -7).all())
