"""The allocation-free signed_bundle entry point (fixed scratch inside the library image),
called through the C ABI and compared with the workspace entry point.

Named so that it is collected last: it must give the same answers on a fresh process and after
every other test has used the library.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _case(seed, B, M, N, D):
    g = torch.Generator().manual_seed(seed)
    W = torch.randint(-128, 128, (B, M, N), generator=g, dtype=torch.int64).to(torch.int8).to(DEV)
    bits = (torch.rand((B, N, D), generator=g) < 0.5).to(DEV)
    return W, torch.ops.brute.pack_bool(bits)


def test_static_scratch_matches_workspace_entry_twice_in_a_row(lib_built):
    import brute_b200  # noqa: F401
    from brute_b200 import _lib as L
    lib = L.load()
    st = torch.cuda.current_stream().cuda_stream
    cap = int(lib.brute_b200_signed_bundle_static_max_bytes())
    assert cap == 1 << 20
    # two calls back to back with different shapes and data: the second must not see the first's scratch
    for seed, (B, M, N, D) in enumerate([(4, 200, 512, 128), (2, 128, 1024, 70), (4, 200, 512, 128)]):
        W, vp = _case(seed, B, M, N, D)
        Dp = vp.size(2)
        need = int(lib.brute_b200_signed_bundle_workspace_bytes(B, N, D))
        assert need <= cap
        want = torch.zeros((B, M, Dp), dtype=torch.int64, device=DEV)
        ws = torch.empty(need // 8, dtype=torch.int64, device=DEV)
        assert lib.brute_b200_signed_bundle_ws(W.data_ptr(), vp.data_ptr(), want.data_ptr(), B, M, N, Dp, D,
                                               ws.data_ptr(), need, st) == 0
        got = torch.full((B, M, Dp), -1, dtype=torch.int64, device=DEV)
        before = torch.cuda.memory_allocated()
        assert lib.brute_b200_signed_bundle_static(W.data_ptr(), vp.data_ptr(), got.data_ptr(), B, M, N, Dp, D, st) == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(got, want), (B, M, N, D)
        # the workspace entry shares the transpose and the kernel with the static one: the oracle
        # is the independent check
        from oracle import c_oracle as co
        assert np.array_equal(got.cpu().numpy().view(np.uint64),
                              co.signed_bundle(W.cpu().numpy(), vp.cpu().numpy().view(np.uint64), D)), (B, M, N, D)
    assert lib.brute_b200_device_status() == 0


def test_static_scratch_rows_padded_beyond_the_logical_width(lib_built):
    """V rows may carry more words than D needs (Dp > ceil(D/64)); the words past D are output as 0."""
    import brute_b200  # noqa: F401
    from brute_b200 import _lib as L
    from oracle import c_oracle as co
    lib = L.load()
    st = torch.cuda.current_stream().cuda_stream
    B, M, N, D, Dp = 2, 128, 256, 64, 2
    g = torch.Generator().manual_seed(11)
    W = torch.randint(-128, 128, (B, M, N), generator=g, dtype=torch.int64).to(torch.int8).to(DEV)
    vp = torch.randint(-2 ** 62, 2 ** 62, (B, N, Dp), generator=g, dtype=torch.int64).to(DEV)   # junk in the padding word
    want = co.signed_bundle(W.cpu().numpy(), vp.cpu().numpy().view(np.uint64), D)
    ws = torch.empty(max(int(lib.brute_b200_signed_bundle_workspace_bytes(B, N, D)), 8) // 8, dtype=torch.int64, device=DEV)
    for entry in ("static", "ws"):
        got = torch.full((B, M, Dp), -1, dtype=torch.int64, device=DEV)
        if entry == "static":
            rc = lib.brute_b200_signed_bundle_static(W.data_ptr(), vp.data_ptr(), got.data_ptr(), B, M, N, Dp, D, st)
        else:
            rc = lib.brute_b200_signed_bundle_ws(W.data_ptr(), vp.data_ptr(), got.data_ptr(), B, M, N, Dp, D,
                                                 ws.data_ptr(), ws.numel() * 8, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint64), want), entry
    assert np.array_equal(torch.ops.brute.signed_bundle(W, vp, D).cpu().numpy().view(np.uint64), want)


def test_static_scratch_on_every_visible_device(lib_built):
    """The array's address is looked up once per device, with that device current."""
    import brute_b200  # noqa: F401
    from brute_b200 import _lib as L
    from oracle import c_oracle as co
    lib = L.load()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    B, M, N, D = 2, 128, 512, 128
    for dev in (1, 0, 1):
        with torch.cuda.device(dev):
            g = torch.Generator().manual_seed(20 + dev)
            W = torch.randint(-128, 128, (B, M, N), generator=g, dtype=torch.int64).to(torch.int8).to(f"cuda:{dev}")
            vp = torch.ops.brute.pack_bool((torch.rand((B, N, D), generator=g) < 0.5).to(f"cuda:{dev}"))
            got = torch.zeros((B, M, vp.size(2)), dtype=torch.int64, device=f"cuda:{dev}")
            st = torch.cuda.current_stream().cuda_stream
            assert lib.brute_b200_signed_bundle_static(W.data_ptr(), vp.data_ptr(), got.data_ptr(), B, M, N,
                                                       vp.size(2), D, st) == 0
            torch.cuda.synchronize()
            assert np.array_equal(got.cpu().numpy().view(np.uint64),
                                  co.signed_bundle(W.cpu().numpy(), vp.cpu().numpy().view(np.uint64), D))


def test_static_scratch_rejects_what_does_not_fit(lib_built):
    import brute_b200  # noqa: F401
    from brute_b200 import _lib as L
    lib = L.load()
    st = torch.cuda.current_stream().cuda_stream
    B, M, N, D = 8, 128, 4096, 300          # 8 * 300 * 64 words * 8 B = 1.17 MiB of scratch
    assert int(lib.brute_b200_signed_bundle_workspace_bytes(B, N, D)) > int(lib.brute_b200_signed_bundle_static_max_bytes())
    W, vp = _case(5, B, M, N, D)
    out = torch.full((B, M, vp.size(2)), 7, dtype=torch.int64, device=DEV)
    rc = lib.brute_b200_signed_bundle_static(W.data_ptr(), vp.data_ptr(), out.data_ptr(), B, M, N, vp.size(2), D, st)
    assert rc == L.ERR_WORKSPACE
    torch.cuda.synchronize()
    assert bool((out == 7).all())           # nothing was launched
    # a shape the tensor path does not take needs no scratch and still answers, whatever its size
    W2, v2 = _case(6, 1, 5, 7, 70)
    out2 = torch.zeros((1, 5, 2), dtype=torch.int64, device=DEV)
    assert lib.brute_b200_signed_bundle_static(W2.data_ptr(), v2.data_ptr(), out2.data_ptr(), 1, 5, 7, 2, 70, st) == 0
    from oracle import c_oracle as co
    assert np.array_equal(out2.cpu().numpy().view(np.uint64), co.signed_bundle(W2.cpu().numpy(), v2.cpu().numpy().view(np.uint64), 70))
