"""Streams and CUDA graphs around the ops (reference: tests/unit/test_streams.py,
brute/streams.py, brute/cuda_graphs.py): every launcher enqueues on the caller's
current stream and never synchronises, so it composes with side streams, the
round-robin pool and graph capture."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def brute(lib_built):
    import brute_b200
    return brute_b200


def test_op_on_side_stream(brute):
    stream = torch.cuda.Stream()
    x = brute.randint(0, 2, (1024, 1024), dtype=brute.bit1, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        y = brute.logical_not(x) if hasattr(brute, "logical_not") else torch.logical_not(x)
    torch.cuda.synchronize()
    assert y.device.type == "cuda" and int(y.popcount()) == x.numel() - int(x.popcount())


def test_event_record_wait(brute):
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    x = brute.randint(0, 2, (128,), dtype=brute.bit1, device="cuda")
    torch.cuda.synchronize()
    evt = torch.cuda.Event()
    with torch.cuda.stream(s1):
        y = torch.logical_not(x)
        evt.record(s1)
    with torch.cuda.stream(s2):
        evt.wait(s2)
        z = torch.logical_not(y)
    torch.cuda.synchronize()
    assert z.dtype == brute.bit1 and torch.equal(z, x)


def test_parallel_streams_pool(brute):
    a = brute.randint(0, 2, (512, 4096), dtype=brute.bit1, device="cuda")
    b = brute.randint(0, 2, (512, 4096), dtype=brute.bit1, device="cuda")
    torch.cuda.synchronize()
    with brute.parallel_streams(4) as rot:
        r1 = a & b
        r2 = a | b
        r3 = a ^ b
        r4 = ~a
        assert len(rot.streams) == 4
        from brute_b200 import ops as _o
        if _o.BINDING == "ctypes":            # this binding's ops really run on the pool streams
            assert rot.idx != 0 or len(rot._tail) > 0
    torch.cuda.synchronize()
    ab, bb = a.bool().as_subclass(torch.Tensor), b.bool().as_subclass(torch.Tensor)
    for got, want in ((r1, ab & bb), (r2, ab | bb), (r3, ab ^ bb), (r4, ~ab)):
        assert torch.equal(got.bool().as_subclass(torch.Tensor), want)


def _bools(brute, shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = torch.rand(shape, device="cuda", generator=g) < 0.5
    return t, brute.Tensor(t, dtype=brute.bit1)


def test_parallel_streams_dependent_chain_and_freed_temporaries(brute):
    """Inside the block every op runs on another stream. A chain must still see its producer's
    result, and a temporary freed in the middle of the chain must not be handed to a later op while
    its reader is still queued."""
    shape = (2048, 4096 + 13)
    xb, x = _bools(brute, shape, 1)
    yb, y = _bools(brute, shape, 2)
    zb, z = _bools(brute, shape, 3)
    want = ((xb & yb) ^ zb) | ~xb
    torch.cuda.synchronize()
    for _ in range(20):
        with brute.parallel_streams(4):
            r = (x & y) ^ z                 # (x & y) is freed as soon as the xor is queued
            r = r | ~x
            junk = [(x ^ y) for _ in range(3)]      # same-size blocks the allocator can recycle
            del junk
            total = r.popcount()
        assert int(total) == int(want.sum())
        assert torch.equal(r.bool().as_subclass(torch.Tensor), want)


def test_parallel_streams_with_plain_torch_ops_between(brute):
    """randn -> pack_sign (a plain torch producer), and a plain torch consumer of a packed result."""
    torch.cuda.synchronize()
    for i in range(10):
        with brute.parallel_streams(3):
            f = torch.randn((1024, 2048), device="cuda")
            b = brute.Tensor(f, dtype=brute.bit1)           # pack_sign on a pool stream
            inv = ~b
            words = torch.bitwise_and(inv._packed_buf, b._packed_buf)     # plain torch on the caller's stream
            col = inv[:, 5]                                  # goes through the bool view
        torch.cuda.synchronize()
        assert torch.equal(b.bool().as_subclass(torch.Tensor), f > 0)
        assert int(words.ne(0).sum()) == 0
        assert torch.equal(col.bool().as_subclass(torch.Tensor), ~(f[:, 5] > 0))


def test_parallel_streams_two_signed_bundles_in_a_row(brute):
    """Both calls allocate a workspace; on different streams they must not share it."""
    from oracle import c_oracle as co
    g = torch.Generator().manual_seed(5)
    W1 = torch.randint(-128, 128, (2, 128, 256), generator=g, dtype=torch.int64).to(torch.int8)
    W2 = torch.randint(-128, 128, (2, 128, 256), generator=g, dtype=torch.int64).to(torch.int8)
    v1 = torch.rand((2, 256, 128), generator=g) < 0.5
    v2 = torch.rand((2, 256, 128), generator=g) < 0.5
    p1, p2 = torch.ops.brute.pack_bool(v1.cuda()), torch.ops.brute.pack_bool(v2.cuda())
    W1c, W2c = W1.cuda(), W2.cuda()
    want1 = co.signed_bundle(W1.numpy(), co.pack_bool(v1.numpy()), 128)
    want2 = co.signed_bundle(W2.numpy(), co.pack_bool(v2.numpy()), 128)
    torch.cuda.synchronize()
    for _ in range(10):
        with brute.parallel_streams(2):
            o1 = torch.ops.brute.signed_bundle(W1c, p1, 128)
            o2 = torch.ops.brute.signed_bundle(W2c, p2, 128)
        torch.cuda.synchronize()
        assert np.array_equal(o1.cpu().numpy().view(np.uint64), want1)
        assert np.array_equal(o2.cpu().numpy().view(np.uint64), want2)


def test_parallel_streams_restores_the_current_stream(brute):
    before = torch.cuda.current_stream()
    x = brute.randint(0, 2, (64, 64), dtype=brute.bit1, device="cuda")
    with brute.parallel_streams(2):
        _ = x & x
        with pytest.raises(RuntimeError):
            torch.ops.brute.bitwise_packed(x._packed_buf, x._packed_buf.cpu(), 0, 64)   # mixed devices: raises, no launch
        _ = x | x
    assert torch.cuda.current_stream() == before
    assert torch.cuda.current_stream is brute.streams._REAL_CURRENT_STREAM


def test_cuda_graph_capture_replay(brute):
    M, K, N = 256, 1024, 512
    a = brute.randint(0, 2, (M, K), dtype=brute.bit1, device="cuda")
    w = brute.randint(0, 2, (N, K), dtype=brute.bit1, device="cuda")
    pa, pw = a._packed_buf, w._packed_buf
    want = brute.matmul_packed(pa, pw, K).clone()
    g = brute.cuda_graphs.capture(lambda: brute.matmul_packed(pa, pw, K), warmup=2)
    # change the operand in place, replay: the captured kernel reads the new bits
    pa.copy_(torch.bitwise_not(pa))
    out = brute.cuda_graphs.replay(g)
    torch.cuda.synchronize()
    assert torch.equal(out, -want)
    from brute_b200 import _lib as L
    assert L.load().brute_b200_device_status() == 0


def test_two_devices_guard(brute):
    # the binding installs a device guard (the reference has none): an op on cuda:1 tensors
    # must run on cuda:1 whatever the current device is
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x = torch.rand((64, 200), device="cuda:1") < 0.5
    with torch.cuda.device(0):
        p = torch.ops.brute.pack_bool(x)
        assert p.device == x.device
        assert int(torch.ops.brute.packed_popcount(p)) == int(x.sum())
