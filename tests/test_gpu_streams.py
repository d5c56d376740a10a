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
    torch.cuda.synchronize()
    ab, bb = a.bool().as_subclass(torch.Tensor), b.bool().as_subclass(torch.Tensor)
    for got, want in ((r1, ab & bb), (r2, ab | bb), (r3, ab ^ bb), (r4, ~ab)):
        assert torch.equal(got.bool().as_subclass(torch.Tensor), want)


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
