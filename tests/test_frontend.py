"""The front end (brute.Tensor, factories, fast helpers) against torch.bool.

Every test runs twice: on CUDA tensors (marked gpu; the product's kernels) and on
CPU tensors. The product has CUDA kernels only; for the CPU run the CPU dispatch
key of torch.ops.brute.* is bound to the oracle (tests/conftest.py) so that the
subclass state machine -- lazy bool storage, version-tracked re-pack,
packed-domain fast paths, the t() source for matmul -- is exercised without a GPU.
The checker is torch.bool itself, as in the reference's op catalog
(tests/ops_catalog.py): run the same function on a bool tensor and on the bit1
tensor and compare.
"""
import copy
import io
import pickle

import numpy as np
import pytest
import torch

DEV = "cpu"


@pytest.fixture(scope="module", params=["cpu", pytest.param("cuda", marks=pytest.mark.gpu)], autouse=True)
def device(request, lib_built):
    global DEV
    if request.param == "cpu":
        import conftest
        conftest.install_oracle_cpu_ops()
    DEV = request.param
    yield request.param
    DEV = "cpu"


@pytest.fixture(scope="module")
def brute(device):
    import brute_b200
    return brute_b200


def b1(brute, t):
    return brute.Tensor(t, dtype=brute.bit1)


def as_bool(x):
    """Plain CPU bool view of a brute tensor (materialises a lazy one)."""
    if hasattr(x, "_ensure_bool_valid"):
        x._ensure_bool_valid()
        x = x.as_subclass(torch.Tensor)
    return x.cpu() if isinstance(x, torch.Tensor) else x


def rnd(shape, seed=0, p=0.5):
    """Seeded bool tensor on the device under test (generated on the CPU so both runs see the same bits)."""
    return (torch.rand(shape, generator=torch.Generator().manual_seed(seed)) < p).to(DEV)


def cpu(t):
    return t.as_subclass(torch.Tensor).cpu() if isinstance(t, torch.Tensor) else t


def same(a, b):
    """torch.equal on CPU copies, so that a materialised view and its torch.bool twin can sit on any device."""
    return torch.equal(cpu(a), cpu(b))


SHAPES = [(16,), (4, 8), (3, 13), (13,), (2, 3, 65), (5, 64), (2, 128)]


def test_dtype_sentinel(brute):
    assert repr(brute.bit1) == "brute.bit1" and str(brute.bit1) == "bit1"
    assert brute.bit1 == type(brute.bit1)() and hash(brute.bit1) == hash(type(brute.bit1)())
    x = b1(brute, rnd((4, 8)))
    assert x.dtype == brute.bit1 and x.type() == "brute.Bit1Tensor"
    with pytest.raises(TypeError):
        x.element_size()
    with pytest.raises(TypeError):
        x.itemsize
    assert x.nbytes == 4 * 8          # 4 rows x 1 word


def test_float_threshold_known_answer(brute):
    # reference tests/unit/test_dtype.py:79-83: [-1, 0, 0.5, 1] -> [F, F, T, T]
    x = brute.tensor([-1.0, 0.0, 0.5, 1.0], dtype=torch.float32, device=DEV).to(brute.bit1)
    assert same(as_bool(x), torch.tensor([False, False, True, True]))
    y = brute.tensor([0, 1, 0, 1, 1], dtype=torch.int32, device=DEV).to(brute.bit1)
    assert same(as_bool(y), torch.tensor([False, True, False, True, True]))


def test_unpack_pm1_known_answer(brute):
    a = brute.tensor([True, False, True, True, False], dtype=brute.bit1, device=DEV)
    assert same(a.unpack_pm1(), torch.tensor([1.0, -1.0, 1.0, 1.0, -1.0]))


@pytest.mark.parametrize("shape", SHAPES)
def test_roundtrip_and_reductions(brute, shape):
    src = rnd(shape, 1)
    x = b1(brute, src)
    assert same(as_bool(x.bool()), src)
    assert int(x.popcount()) == int(src.sum()) == int(x.sum()) == int(torch.count_nonzero(x))
    assert int(x.word_popcount().as_subclass(torch.Tensor).long().sum()) == int(src.sum())
    assert bool(torch.any(x)) == bool(src.any()) and bool(torch.all(x)) == bool(src.all())
    assert same(as_bool(torch.any(x, dim=-1)), src.any(dim=-1))
    assert same(as_bool(torch.all(x, -1)), src.all(dim=-1))
    if len(shape) >= 2:
        assert same(as_bool(x.any(dim=0)), src.any(dim=0))
        assert same(as_bool(x.all(dim=0, keepdim=True)), src.all(dim=0, keepdim=True))


@pytest.mark.parametrize("shape", SHAPES)
def test_bitwise_parity_with_bool(brute, shape):
    sa, sb, sc = rnd(shape, 2), rnd(shape, 3), rnd(shape, 4)
    a, b, c = b1(brute, sa), b1(brute, sb), b1(brute, sc)
    cases = {
        "and": (a & b, sa & sb), "or": (a | b, sa | sb), "xor": (a ^ b, sa ^ sb), "not": (~a, ~sa),
        "f_and": (torch.bitwise_and(a, b), sa & sb), "l_or": (torch.logical_or(a, b), sa | sb),
        "l_xor": (a.logical_xor(b), sa ^ sb), "l_not": (torch.logical_not(a), ~sa),
        "eq": (a == b, sa == sb), "ne": (torch.ne(a, b), sa != sb),
        "where": (torch.where(c, a, b), torch.where(sc, sa, sb)),
        "fast_eq": (brute.eq(a, b), sa == sb), "fast_xor": (brute.bitwise_xor(a, b), sa ^ sb),
        "fast_not": (brute.bitwise_not(a), ~sa),
    }
    for name, (got, want) in cases.items():
        assert got.dtype == brute.bit1, name
        assert got.__dict__.get("_bool_dirty") is True, f"{name}: packed-domain result should be lazy"
        assert same(as_bool(got), want), name
        assert int(got.popcount()) == int(want.sum()), f"{name}: pad bits leaked"
    assert int(a.hamming(b)) == int((sa ^ sb).sum()) == int(brute.hamming(a, b))
    assert torch.equal(a, a.clone()) and (not torch.equal(a, ~a) or a.numel() == 0)


def test_operator_fast_paths_fall_back(brute):
    # ==, !=, ^, &, | skip __torch_function__ for two bit1 tensors of one shape; everything else
    # (scalars, plain bool tensors, broadcasting, 0-dim) must take the general path and agree with torch
    sa, sb = rnd((3, 70), 5), rnd((3, 70), 6)
    a, b = b1(brute, sa), b1(brute, sb)
    assert (a != b).dtype == brute.bit1 and same(as_bool(a != b), sa != sb)
    assert same(as_bool(a == b), sa == sb)
    row = b1(brute, sb[0])                                  # broadcast: general path
    assert same(as_bool(a ^ row), sa ^ sb[0]) and same(as_bool(a == row), sa == sb[0])
    plain = sb.clone()                                      # a plain bool operand does not promote
    assert same(cpu(a == plain), sa == sb) and same(cpu(a & plain), sa & sb)
    assert same(cpu(a == True), sa == True)                 # noqa: E712  (scalar comparison)
    z0, z1 = b1(brute, sa[0, 0]), b1(brute, sb[0, 0])       # 0-dim
    assert bool(cpu(z0 == z1)) == bool(sa[0, 0] == sb[0, 0])
    assert hash(a) == hash(a) and a in [a] and len({a: 1, b: 2}) == 2   # defining __eq__ kept the hash
    # nested and keyword arguments reach the handlers through the hand-rolled flattener
    assert same(as_bool(torch.cat([a, b], dim=0)), torch.cat([sa, sb], dim=0))
    assert same(as_bool(torch.stack((a, b))), torch.stack((sa, sb)))
    assert same(as_bool(torch.where(condition=a, input=b, other=a)), torch.where(sa, sb, sa))
    assert same(as_bool(torch.cat(tensors=[a, b], dim=1)), torch.cat([sa, sb], dim=1))
    parts = torch.split(a, [1, 2], dim=0)
    assert same(as_bool(parts[1]), sa[1:])


def test_invert_pad_safe_sizes(brute):
    for n in [1, 7, 8, 9, 31, 32, 33, 63, 64, 65, 1003, 4096]:
        src = rnd((n,), n)
        inv = ~b1(brute, src)
        assert int(inv.popcount()) == n - int(src.sum())
        assert same(as_bool(inv), ~src)


def test_inplace_ops_touch_only_packed(brute):
    sa, sb = rnd((3, 70), 5), rnd((3, 70), 6)
    a, b = b1(brute, sa), b1(brute, sb)
    a &= b
    assert a.__dict__["_bool_dirty"] is True
    assert same(as_bool(a), sa & sb)
    a |= b
    a ^= b
    assert same(as_bool(a), ((sa & sb) | sb) ^ sb)


def test_version_counter_repacks_after_bool_write(brute):
    src = rnd((4, 70), 7)
    x = b1(brute, src.clone())
    before = x._packed_buf.clone()
    x.as_subclass(torch.Tensor)[1, 3] = not bool(src[1, 3])        # write through the bool storage
    after = x._packed_buf
    assert not torch.equal(before, after)
    src2 = src.clone()
    src2[1, 3] = not bool(src[1, 3])
    assert int(x.popcount()) == int(src2.sum())
    x.fill_(True)
    assert int(x.popcount()) == x.numel() and bool(as_bool(x).all())
    x.zero_()
    assert int(x.popcount()) == 0


def test_lazy_bool_materialises_once(brute):
    a, b = b1(brute, rnd((5, 65), 8)), b1(brute, rnd((5, 65), 9))
    c = a ^ b
    assert c.__dict__["_bool_dirty"] is True
    _ = c.shape, c.dim(), c.device                       # metadata never unpacks
    assert c.__dict__["_bool_dirty"] is True
    _ = c + 0                                             # a generic op does
    assert c.__dict__["_bool_dirty"] is False
    assert same(as_bool(c), as_bool(a) ^ as_bool(b))


@pytest.mark.parametrize("shape", [(4, 64), (3, 13), (2, 3, 128), (2, 5, 7)])
def test_view_ops_parity(brute, shape):
    src = rnd(shape, 10)
    x = b1(brute, src)
    fns = [
        lambda t: t.reshape(-1), lambda t: t.flatten(), lambda t: t.ravel(), lambda t: t.clone(),
        lambda t: t.unsqueeze(0), lambda t: t.unsqueeze(-1), lambda t: t.unsqueeze(0).squeeze(0),
        lambda t: t.transpose(0, -1), lambda t: t.transpose(0, 0), lambda t: t.detach(),
        lambda t: t.permute(*reversed(range(t.dim()))), lambda t: t.contiguous(),
        lambda t: t.movedim(0, -1), lambda t: torch.flip(t, [0]), lambda t: t[0], lambda t: t[1:],
        lambda t: t.view(t.shape), lambda t: t.repeat(*([2] + [1] * (t.dim() - 1))),
        lambda t: torch.index_select(t, 0, torch.tensor([1, 0, 1], device=DEV)),
        lambda t: t.repeat_interleave(2, dim=0),
    ]
    if len(shape) >= 3:
        fns += [lambda t: t.transpose(0, 1), lambda t: t.permute(1, 0, 2), lambda t: torch.swapaxes(t, 0, 1),
                lambda t: torch.movedim(t, 0, 1), lambda t: torch.fliplr(t), lambda t: torch.flipud(t)]
    for i, fn in enumerate(fns):
        got, want = fn(x), fn(src)
        assert got.dtype == brute.bit1, i
        assert tuple(got.shape) == tuple(want.shape), i
        assert same(as_bool(got), want), i
        assert int(got.popcount()) == int(want.sum()), i


def test_setitem_fast_paths(brute):
    src = rnd((6, 70), 11)
    x = b1(brute, src.clone())
    ref = src.clone()
    x[2] = True; ref[2] = True
    x[4:6] = False; ref[4:6] = False
    x[:, 69] = True; ref[:, 69] = True
    x[..., 3] = False; ref[..., 3] = False
    x[0, 5] = True; ref[0, 5] = True                      # generic path
    assert same(as_bool(x), ref) and int(x.popcount()) == int(ref.sum())
    with pytest.raises(IndexError):
        x[:, 70] = True


def test_matmul_paths(brute):
    M, K, N = 5, 130, 7
    sa, sb = rnd((M, K), 12), rnd((N, K), 13)
    a, b = b1(brute, sa), b1(brute, sb)
    want = ((sa.float() * 2 - 1) @ (sb.float() * 2 - 1).t()).to(torch.int32)
    assert same(a @ b, want)                        # B stored (N, K)
    assert same(a @ b.t(), want)                    # via _t_source
    assert same(torch.matmul(a, b.t()), want)
    assert same(torch.mm(a, b.transpose(0, 1)), want)
    assert same(brute.matmul(a, b), want)
    assert same(brute.matmul_packed(a._packed_buf, b._packed_buf, K), want)
    assert (a @ b).dtype == torch.int32 and not isinstance(a @ b, brute.Tensor)


def test_factories(brute):
    for size in [(5,), (3, 70), (2, 64)]:
        z, o = brute.zeros(*size, dtype=brute.bit1, device=DEV), brute.ones(size, dtype=brute.bit1, device=DEV)
        assert int(z.popcount()) == 0 and int(o.popcount()) == int(np.prod(size))
        assert bool(as_bool(o).all()) and not bool(as_bool(z).any())
        e = brute.empty(*size, dtype=brute.bit1, device=DEV)
        assert int(e.popcount()) <= int(np.prod(size))
        f = brute.full(size, 1, dtype=brute.bit1, device=DEV)
        assert int(f.popcount()) == int(np.prod(size))
    g = torch.Generator(device=DEV).manual_seed(3)
    r = brute.randn(4, 100, dtype=brute.bit1, generator=g, device=DEV)
    ref = torch.randn(4, 100, generator=torch.Generator(device=DEV).manual_seed(3), device=DEV) >= 0
    assert same(as_bool(r), ref)
    ri = brute.randint(0, 2, (128,), dtype=brute.bit1, device=DEV)
    assert ri.dtype == brute.bit1 and 0 <= int(ri.popcount()) <= 128
    assert brute.zeros_like(r).dtype == brute.bit1 and brute.ones_like(r, dtype=torch.float32).dtype == torch.float32
    assert isinstance(brute.arange(5), brute.Tensor) and brute.nn is None and brute.optim is None


def test_randomize_keeps_pad_bits_zero(brute):
    a = brute.zeros(3, 1003, dtype=brute.bit1, device=DEV)
    a.randomize_()
    assert 0 < int(a.popcount()) < 3 * 1003
    assert int(a.popcount()) == int(as_bool(a.bool()).sum())


def test_type_errors(brute):
    a = brute.zeros(8, dtype=brute.bit1, device=DEV)
    plain = torch.zeros(8, dtype=torch.bool, device=DEV).as_subclass(brute.Tensor)
    with pytest.raises(TypeError):
        a.hamming(torch.zeros(8, dtype=torch.bool, device=DEV))
    with pytest.raises(ValueError):
        a.hamming(brute.zeros(16, dtype=brute.bit1, device=DEV))
    for fn in (lambda: plain.word_popcount(), lambda: plain.randomize_(), lambda: plain.unpack_pm1()):
        with pytest.raises(TypeError):
            fn()
    assert int(brute.Tensor(torch.ones(4, dtype=torch.bool, device=DEV)).popcount()) == 4


def test_mixed_bool_does_not_promote(brute):
    sa, sb = rnd((4, 9), 14), rnd((4, 9), 15)
    out = torch.logical_and(b1(brute, sa), sb)
    assert out.dtype == torch.bool and same(out, sa & sb)
    picked = b1(brute, sa)[sb]                           # mask indexing keeps bit1
    assert picked.dtype == brute.bit1
    assert int(torch.argmax(b1(brute, sa).flatten())) == int(torch.argmax(sa.flatten().to(torch.uint8)))


def test_pickle_deepcopy_numpy_repr(brute):
    src = rnd((3, 70), 16)
    x = b1(brute, src) ^ b1(brute, torch.zeros_like(src))          # a lazy one
    y = pickle.loads(pickle.dumps(x))
    assert y.dtype == brute.bit1 and same(as_bool(y), src)
    buf = io.BytesIO()
    torch.save(x, buf)
    buf.seek(0)
    z = torch.load(buf, weights_only=False)
    assert same(as_bool(z), src)
    d = copy.deepcopy(x)
    assert d.dtype == brute.bit1 and same(as_bool(d), src) and int(d.popcount()) == int(src.sum())
    assert np.array_equal(np.asarray(x), src.cpu().numpy())
    assert "brute.Tensor(" in repr(x) and "dtype=brute.bit1" in repr(x)


def test_empty_and_zero_dim(brute):
    for shape in [(0,), (3, 0), (0, 5)]:
        x = b1(brute, torch.zeros(shape, dtype=torch.bool, device=DEV))
        assert tuple(x.shape) == shape and int(x.popcount()) == 0
    s = brute.Tensor(torch.tensor(True, device=DEV), dtype=brute.bit1)
    assert s.dim() == 0 and int(s.popcount()) == 1 and bool(as_bool(~s)) is False


# ---------------------------------------------------------------------------
# packed serialisation, packed-domain transpose and leading-axis reductions
# ---------------------------------------------------------------------------
def test_save_load_packed_roundtrip(brute, tmp_path):
    x = rnd((37, 1003), 11)
    y = rnd((5,), 12)
    state = {"w": b1(brute, x), "nested": [b1(brute, y), torch.arange(4)], "step": 7}
    path = tmp_path / "state.pt"
    brute.save_packed(state, path)
    back = brute.load_packed(path, device=DEV)
    assert back["step"] == 7 and torch.equal(cpu(back["nested"][1]), torch.arange(4))
    assert back["w"].dtype == brute.bit1 and tuple(back["w"].shape) == (37, 1003)
    assert str(back["w"].device).startswith(DEV)
    assert torch.equal(as_bool(back["w"]), x.cpu()) and torch.equal(as_bool(back["nested"][0]), y.cpu())
    # 64 bits per stored word instead of 8 per bool byte
    bool_path = tmp_path / "bool.pt"
    torch.save({"w": x.cpu()}, bool_path)
    assert path.stat().st_size < bool_path.stat().st_size / 5
    with pytest.raises(ValueError, match="reserved"):
        brute.save_packed({"__bit1__": 1}, tmp_path / "bad.pt")


def test_transpose_keeps_packed_domain(brute):
    x = rnd((3, 70, 130), 13)
    b = b1(brute, x)
    for dims in ((-1, -2), (1, 2)):
        bt = b.transpose(*dims)
        assert tuple(bt.shape) == (3, 130, 70)
        assert torch.equal(as_bool(bt), x.transpose(*dims).cpu())
        want = torch.ops.brute.pack_bool(x.transpose(*dims).contiguous())
        assert torch.equal(bt._packed_buf, want)
    m = rnd((65, 129), 14)
    assert torch.equal(as_bool(b1(brute, m).t() ^ b1(brute, m.t().contiguous())), torch.zeros(129, 65, dtype=torch.bool))


def test_any_all_over_leading_dims(brute):
    x = rnd((6, 9, 131), 15, p=0.8)
    b = b1(brute, x)
    for dim in (0, 1, -2, -3):
        for keepdim in (False, True):
            assert torch.equal(as_bool(b.any(dim=dim, keepdim=keepdim)), x.any(dim=dim, keepdim=keepdim).cpu())
            assert torch.equal(as_bool(b.all(dim=dim, keepdim=keepdim)), x.all(dim=dim, keepdim=keepdim).cpu())


def test_flip_roll_index_select_on_packed_axis(brute):
    x = rnd((3, 5, 131), 16)
    b = b1(brute, x)
    cases = {
        "flip_last": (torch.flip(b, [-1]), torch.flip(x, [-1])),
        "flip_all": (b.flip(0, 2), x.flip(0, 2)),
        "roll_last": (torch.roll(b, 7, -1), torch.roll(x, 7, -1)),
        "roll_neg": (b.roll(-200, 2), x.roll(-200, 2)),
        "roll_two": (torch.roll(b, (1, 70), (0, -1)), torch.roll(x, (1, 70), (0, -1))),
    }
    idx = torch.tensor([130, 0, 5, 5, 64, 63], device=DEV)
    cases["index_select"] = (torch.index_select(b, -1, idx), torch.index_select(x, -1, idx))
    for name, (got, want) in cases.items():
        assert got.dtype == brute.bit1 and tuple(got.shape) == tuple(want.shape), name
        assert got.__dict__.get("_bool_dirty") is True, f"{name}: should stay in the packed domain"
        assert same(as_bool(got), want), name
        assert int(got.popcount()) == int(want.sum()), f"{name}: pad bits leaked"
    with pytest.raises(IndexError):
        torch.index_select(b, -1, torch.tensor([131], device=DEV))
    rep = b.repeat(2, 1, 3)
    assert rep.__dict__.get("_bool_dirty") is True, "repeat of a ragged last dim should stay packed"
    assert same(as_bool(rep), x.repeat(2, 1, 3)) and int(rep.popcount()) == int(x.repeat(2, 1, 3).sum())
    # a slice of the packed axis is a VIEW in torch (a write through it reaches the base), so it is a
    # bool view here as in the reference (brute/tensor.py:846-853), not a packed-domain copy
    for name, got, want in (("slice", b[..., 3:100], x[..., 3:100]), ("slice_step", b[:, :, 1::3], x[:, :, 1::3]),
                            ("slice_neg", b[..., -70:-1:2], x[..., -70:-1:2])):
        assert got.dtype == brute.bit1 and tuple(got.shape) == tuple(want.shape), name
        assert same(as_bool(got), want), name
        assert int(got.popcount()) == int(want.sum()), f"{name}: pad bits leaked"
    assert same(as_bool(b[..., 5:5]), x[..., 5:5])          # empty: the generic path


# ---------------------------------------------------------------------------
# a packed-only (lazy) result must behave like the reference's, which owns real bool storage
# (brute/tensor.py:288-352): strides, in-place fills, aliasing; and it must cost no memory until read
# ---------------------------------------------------------------------------
def test_lazy_result_reports_contiguous_strides(brute):
    # reference tests/unit/test_layout.py:46
    z = brute.zeros((3, 4, 5), dtype=brute.bit1, device=DEV)
    assert z.stride() == (20, 5, 1) and z.stride(0) == 20 and z.stride(-1) == 1
    assert z.is_contiguous() and z.storage_offset() == 0
    y = b1(brute, rnd((2, 1, 7), 3)) ^ b1(brute, rnd((2, 1, 7), 4))
    assert y.__dict__["_bool_dirty"] is True
    assert y.stride() == torch.empty((2, 1, 7)).stride()


def test_fill_and_zero_on_a_lazy_result(brute):
    # reference tests/unit/test_lazy_bool.py:142, tests/stress/test_cache_rebuilds.py:15,
    # catalog specs fill_true / fill_false / zero_ (tests/ops_catalog.py:607-619)
    for shape in ((64,), (3, 13), (2, 3, 65)):
        a, c = rnd(shape, 31), rnd(shape, 32)
        lazy = b1(brute, a) & b1(brute, c)
        assert lazy.__dict__["_bool_dirty"] is True
        out = lazy.fill_(True)
        assert out is lazy and int(lazy.sum()) == lazy.numel()
        assert lazy.__dict__["_bool_dirty"] is True, "a fill of a packed-only tensor must not allocate bool storage"
        assert same(as_bool(lazy), torch.ones(shape, dtype=torch.bool))
        lazy.fill_(False)
        assert int(lazy.popcount()) == 0 and same(as_bool(lazy), torch.zeros(shape, dtype=torch.bool))
        z = brute.ones(shape, dtype=brute.bit1, device=DEV)
        z.zero_()
        assert int(z.sum()) == 0 and same(as_bool(z), torch.zeros(shape, dtype=torch.bool))
    x = brute.zeros(64, dtype=brute.bit1, device=DEV)
    pb0 = x._packed_buf.clone()
    x.fill_(True)
    assert not torch.equal(pb0, x._packed_buf)
    x.fill_(False)
    assert torch.equal(pb0, x._packed_buf)


def test_fill_through_a_view_reaches_the_base(brute):
    # reference tests/unit/test_aliasing.py:15-18,44
    base = brute.zeros((8, 8), dtype=brute.bit1, device=DEV)
    view = base[:, ::2]
    pa = cpu(base).untyped_storage().data_ptr()
    assert cpu(view).untyped_storage().data_ptr() == pa or DEV == "cuda"
    assert base.as_subclass(torch.Tensor).untyped_storage().data_ptr() == \
        view.as_subclass(torch.Tensor).untyped_storage().data_ptr()
    view.fill_(True)
    want = torch.zeros((8, 8), dtype=torch.bool)
    want[:, ::2] = True
    assert same(as_bool(base), want) and int(base.popcount()) == 32
    # the packed buffer of the base follows (version-tracked re-pack)
    assert int(base.sum()) == 32


def test_aliases_taken_before_materialisation_share_storage(brute):
    a, c = rnd((5, 70), 41), rnd((5, 70), 42)
    lazy = b1(brute, a) | b1(brute, c)
    assert lazy.__dict__["_bool_dirty"] is True
    plain_before = torch.Tensor.as_subclass(lazy, torch.Tensor)       # the raw alias: no materialisation
    assert plain_before.untyped_storage().nbytes() == 0, "a lazy result must own no bool storage"
    got = as_bool(lazy)                                               # materialises in place
    assert same(got, a | c)
    assert plain_before.untyped_storage().nbytes() == 5 * 70
    assert torch.equal(plain_before.cpu(), (a | c).cpu()), "an alias taken before the read must see the data"
    assert lazy.stride() == (70, 1)
    # the public as_subclass hands out valid memory, never the empty placeholder
    other = b1(brute, a) ^ b1(brute, c)
    assert torch.equal(other.as_subclass(torch.Tensor).cpu(), (a ^ c).cpu())


def test_large_lazy_result_allocates_no_bool_tensor(brute):
    """2^30 bits: the operands are 128 MiB each; the lazy result may add its 128 MiB of packed words
    but not the 1 GiB bool tensor the reference allocates (brute/tensor.py:316), not even briefly."""
    if DEV != "cuda":
        pytest.skip("needs the CUDA allocator's counters")
    n = 1 << 30
    g = torch.Generator(device="cuda").manual_seed(7)
    pa = torch.randint(-2 ** 62, 2 ** 62, (n // 64,), dtype=torch.int64, device="cuda", generator=g)
    pb = torch.randint(-2 ** 62, 2 ** 62, (n // 64,), dtype=torch.int64, device="cuda", generator=g)
    a = brute.Tensor._make_bit1_from_packed(pa, [n])
    b = brute.Tensor._make_bit1_from_packed(pb, [n])
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    c = (a ^ b) & ~a
    c.fill_(True)
    pop = int(c.popcount())
    torch.cuda.synchronize()
    grown = torch.cuda.memory_allocated() - before
    peak = torch.cuda.max_memory_allocated() - before
    assert pop == n and c.__dict__["_bool_dirty"] is True
    assert c.stride() == (1,) and c.shape == (n,)
    assert grown <= (n // 8) + (1 << 20), f"a lazy result kept {grown} bytes"
    assert peak <= 4 * (n // 8), f"peak {peak} bytes: a bool tensor of 2^30 bytes was allocated on the way"
    # reading it as bool is what allocates
    row = c[:8]
    assert bool(row.all()) and torch.cuda.memory_allocated() - before >= n


def test_move_between_devices_carries_the_packed_words(brute, tmp_path):
    """load_packed() leaves the words on the host; .to('cuda') must move THEM (no CPU kernel exists in
    the product to unpack with) and keep the result packed-only."""
    if DEV != "cuda":
        pytest.skip("needs two device types")
    x = rnd((5, 131), 61)
    b = b1(brute, x) ^ brute.zeros((5, 131), dtype=brute.bit1, device="cuda")
    path = tmp_path / "t.pt"
    brute.save_packed({"w": b}, path)
    host = brute.load_packed(path)["w"]
    assert host._packed_buf.device.type == "cpu" and host.__dict__["_bool_dirty"] is True
    back = host.to("cuda")
    assert back.dtype == brute.bit1 and back.__dict__["_bool_dirty"] is True and back._packed_buf.is_cuda
    assert same(as_bool(back), x) and int(back.popcount()) == int(x.sum())
    assert same(as_bool(brute.load_packed(path, device="cuda")["w"]), x)


def test_clone_then_write_plain_alias_leaves_the_source_alone(brute):
    # reference tests/unit/test_aliasing.py:65-72
    x = brute.zeros(16, dtype=brute.bit1, device=DEV)
    c = x.clone()
    c.as_subclass(torch.Tensor).fill_(True)
    assert same(as_bool(x), torch.zeros(16, dtype=torch.bool))
    assert int(c.popcount()) == 16


# ---------------------------------------------------------------------------
# writes through a tensor index on the packed axis stay in the packed domain
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("state", ["lazy", "valid"])
def test_scatter_on_the_packed_axis(brute, state):
    shape = (5, 3, 131)
    x = rnd(shape, 51)
    idx = torch.tensor([130, 0, 64, 63, 7, 129, -3], device=DEV)        # -3 -> 128
    srcb = rnd(shape[:-1] + (7,), 52)

    def fresh():
        b = b1(brute, x)
        if state == "lazy":
            b = b ^ brute.zeros(shape, dtype=brute.bit1, device=DEV)     # packed-only, bool storage empty
            assert b.__dict__["_bool_dirty"] is True
        return b

    def twin():
        return x.clone()

    # x[..., idx] = scalar
    for v in (True, False):
        b, t = fresh(), twin()
        b[..., idx] = v
        t[..., idx] = v
        assert same(as_bool(b), t) and int(b.popcount()) == int(t.sum())
    # x[:, :, idx] = tensor (bool and bit1 sources)
    for src in (srcb, b1(brute, srcb)):
        b, t = fresh(), twin()
        b[:, :, idx] = src
        t[:, :, idx] = srcb
        assert same(as_bool(b), t) and int(b.popcount()) == int(t.sum())
    # index_fill_ / index_copy_ on the last dim
    b, t = fresh(), twin()
    assert b.index_fill_(-1, idx, True) is b
    t.index_fill_(-1, idx, True)
    assert same(as_bool(b), t)
    b, t = fresh(), twin()
    pos = torch.where(idx < 0, idx + 131, idx)            # torch's index_copy_ takes no negative index
    b.index_copy_(2, pos, b1(brute, srcb))
    t.index_copy_(2, pos, srcb)
    assert same(as_bool(b), t) and int(b.popcount()) == int(t.sum())
    with pytest.raises(IndexError):
        fresh().index_copy_(2, idx, b1(brute, srcb))
    if state == "lazy":
        lz = fresh()
        lz[..., idx] = True
        assert lz.__dict__["_bool_dirty"] is True, "a packed-only tensor must stay packed-only"
    # an index out of range raises before anything is launched
    with pytest.raises(IndexError):
        fresh()[..., torch.tensor([131], device=DEV)] = True
    with pytest.raises(IndexError):
        fresh().index_fill_(-1, torch.tensor([-132], device=DEV), True)


def test_scatter_on_the_packed_axis_reaches_aliases(brute):
    base = b1(brute, rnd((6, 70), 53))
    want = as_bool(base).clone()
    view = base[:, ::2]                      # a bool view that shares base's storage
    base[:, torch.tensor([0, 2, 69], device=DEV)] = True
    want[:, [0, 2, 69]] = True
    assert same(as_bool(base), want)
    assert same(as_bool(view), want[:, ::2]), "the view must see the write"
    assert int(base.popcount()) == int(want.sum())
    # and a write through the plain alias afterwards still re-packs (version tracking intact)
    base.as_subclass(torch.Tensor)[0, 1] = True
    want[0, 1] = True
    assert int(base.popcount()) == int(want.sum())


# ---------------------------------------------------------------------------
# concurrent host threads (the reference requires this of its drivers: tests/unit/test_multithread.py)
# ---------------------------------------------------------------------------
def test_threads_share_one_tensor_and_the_library(brute):
    from concurrent.futures import ThreadPoolExecutor
    src = rnd((64, 300), 21)
    x = b1(brute, src)
    w = b1(brute, rnd((40, 300), 22))
    want_pop = int(src.sum())
    want_mm = cpu(x @ w.t())

    def reader(_):
        # every thread walks the cached packed buffer, makes lazy results, and launches kernels
        acc = 0
        for _ in range(20):
            acc += int(x.popcount())
            y = ~(x ^ x.clone())
            assert int(y.popcount()) == x.numel()
            assert torch.equal(cpu(x @ w.t()), want_mm)
        return acc

    def maker(seed):
        for i in range(20):
            a = b1(brute, rnd((3, 70), 100 + seed * 20 + i))
            b = b1(brute, rnd((3, 70), 500 + seed * 20 + i))
            assert int((a & b).popcount()) + int((a ^ b).popcount()) == int((a | b).popcount())
        return True

    with ThreadPoolExecutor(max_workers=4) as ex:
        got = list(ex.map(reader, range(4)))
        assert all(list(ex.map(maker, range(4))))
    assert got == [20 * want_pop] * 4
