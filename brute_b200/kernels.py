"""Entry points for the parts of the path that the reference composes by hand.

* ``pack_sign``       float -> bit1 in one pass (threshold x > 0 or x >= 0);
* ``binary_linear``   one binarised-MLP layer: xnor GEMM, per-channel fp32
                      scale, re-binarisation, re-pack, fused in the GEMM epilogue;
* ``binary_attention`` sign-binarised Q.K^T scored by popcount, fp32 softmax, @ V;
* ``sharded_matmul``  the xnor GEMM with B's rows (output features) split across
                      the ranks of a ``torch.distributed`` group, optional all-gather;
* ``host_matmul``     the xnor GEMM on operands and a result in HOST memory: the copies in, the
                      GEMM of each block of A's rows and the copy of that block of C back to the
                      host run on three streams and overlap.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .tensor import Tensor, _is_b1

_ops = torch.ops.brute
SIGN_GT0, SIGN_GE0 = 0, 1


def pack_sign(x: torch.Tensor, ge0: bool = False) -> Tensor:
    """Binarise a float tensor into a bit1 tensor: bit = x > 0, or x >= 0 with ``ge0``."""
    base = x.as_subclass(torch.Tensor)
    packed = _ops.pack_sign(base, SIGN_GE0 if ge0 else SIGN_GT0)
    return Tensor._make_bit1_from_packed(packed, list(base.shape))


def binary_linear(x: Tensor, weight: Tensor, scale: torch.Tensor, ge0: bool = True) -> Tensor:
    """bit1 [M, K] x bit1 weight [N, K] -> bit1 [M, N] = sign(scale[n] * (K - 2H))."""
    K = int(x.shape[-1])
    out = _ops.xnor_matmul_scale_sign_pack(x._packed_buf_contig(), weight._packed_buf_contig(),
                                           scale.as_subclass(torch.Tensor), K, SIGN_GE0 if ge0 else SIGN_GT0)
    return Tensor._make_bit1_from_packed(out, [int(x.shape[0]), int(weight.shape[0])])


def binary_attention(q: Tensor, k: Tensor, v: torch.Tensor, causal: bool = True,
                     scale: Optional[float] = None) -> torch.Tensor:
    """q, k bit1 [B, H, S, D]; v bf16 [B, H, S, D] -> bf16 [B, H, S, D]."""
    if not (_is_b1(q) and _is_b1(k)):
        raise TypeError("binary_attention: q and k must be bit1 tensors")
    D = int(q.shape[-1])
    if scale is None:
        scale = D ** -0.5
    return _ops.binary_attention(q._packed_buf_contig(), k._packed_buf_contig(),
                                 v.as_subclass(torch.Tensor), bool(causal), float(scale))


def shard_bounds(n: int, world_size: int, rank: int) -> tuple:
    """Rows [lo, hi) of an n-row operand owned by `rank`: equal blocks, the last
    ranks one row shorter when world_size does not divide n."""
    base, extra = divmod(n, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


_comm_streams = {}


def _comm_stream(dev: torch.device) -> "torch.cuda.Stream":
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _comm_streams:
        # high priority: its kernels take the SMs that a co-running GEMM leaves free as soon as they are due
        _comm_streams[key] = torch.cuda.Stream(dev, priority=-1)
    return _comm_streams[key]


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    """The collective moves bytes; neither NCCL nor gloo has a 16-bit integer type."""
    return t.view(torch.uint8)


def _gather_row_blocks(a_packed, b_local, K: int, world: int, group, row_blocks: Optional[int],
                       leave_sms: int = 32) -> torch.Tensor:
    """The replicated [M, N] result of an evenly column-sharded GEMM, every rank's block exchanged.

    Three things keep the exchange from dominating (at 8 GPUs the plain int32 all-gather of a
    16384^2 result takes five times as long as the rank's GEMM):
    * for K <= 32767 the blocks travel as int16 (|C| <= K fits), half the bytes; the receiver widens
      them while it lays them out, in one pass (``unstack_rank_blocks``);
    * A's rows are cut into blocks: the all-gather of block i runs on a second stream while the GEMM
      of block i+1 runs, ordered by events, no host synchronisation;
    * the GEMM of a block that runs next to a gather leaves ``leave_sms`` SMs free: its persistent
      kernel would otherwise hold every SM and the collective's kernel could only start after it
      (NCCL moves about 30 GB/s per CTA here: 32 SMs carry the full rate of the links).
    On CPU tensors (gloo) the same steps run one after the other.
    """
    import torch.distributed as dist

    M, n_loc = int(a_packed.shape[0]), int(b_local.shape[0])
    dev = a_packed.device
    on_gpu = dev.type == "cuda"
    narrow = int(K) <= 32767
    nb = int(row_blocks) if row_blocks else max(1, min(4, M // 2048))
    nb = max(1, min(nb, M)) if M else 1
    bounds = [shard_bounds(M, nb, i) for i in range(nb)]
    bounds = [(m0, m1) for m0, m1 in bounds if m1 > m0]
    out = torch.empty((M, world * n_loc), dtype=torch.int32, device=dev)
    # scratch of the call, kept between calls of one shape (see release_gather_workspace): this rank's
    # int32 blocks, their int16 form, and the staging area the rank blocks of every row block land in
    c_all, send_all, stage = _gather_workspace(dev, M, n_loc, world, narrow)
    if on_gpu:
        cur = torch.cuda.current_stream(dev)
        comm = _comm_stream(dev)
        comm.wait_stream(cur)
    pending = None                        # (first row, last row, event) of the block whose gather is in flight
    for i, (m0, m1) in enumerate(bounds):
        leave = int(leave_sms) if (on_gpu and i > 0) else 0
        c = _ops.xnor_popcount_matmul_out(a_packed[m0:m1], b_local, K, leave, c_all[m0:m1])
        send = _ops.narrow_i32_i16_out(c, send_all[m0:m1]) if narrow else c
        recv = stage[m0 * world:m1 * world]
        done = None
        if on_gpu:
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                dist.all_gather_into_tensor(_as_bytes(recv), _as_bytes(send), group=group)
                done = torch.cuda.Event()
                done.record(comm)
        else:
            dist.all_gather_into_tensor(_as_bytes(recv), _as_bytes(send), group=group)
        if pending is not None:           # behind this block's GEMM: the previous gather ran under it
            p0, p1, ev = pending
            if on_gpu:
                cur.wait_event(ev)
            _ops.unstack_rank_blocks(stage[p0 * world:p1 * world].view(world, p1 - p0, n_loc), out, p0)
        pending = (m0, m1, done)
    if pending is not None:
        p0, p1, ev = pending
        if on_gpu:
            cur.wait_event(ev)             # the caller's stream is now behind every collective of the call
        _ops.unstack_rank_blocks(stage[p0 * world:p1 * world].view(world, p1 - p0, n_loc), out, p0)
    return out


_gather_ws = {}


def _gather_workspace(dev, M: int, n_loc: int, world: int, narrow: bool):
    key = (str(dev), M, n_loc, world, narrow)
    ws = _gather_ws.get(key)
    if ws is None:
        c_all = torch.empty((M, n_loc), dtype=torch.int32, device=dev)
        send_all = torch.empty((M, n_loc), dtype=torch.int16, device=dev) if narrow else None
        stage = torch.empty((world * M, n_loc), dtype=torch.int16 if narrow else torch.int32, device=dev)
        _gather_ws.clear()                # one shape at a time: a new shape replaces the old scratch
        ws = _gather_ws[key] = (c_all, send_all, stage)
    return ws


# ---------------------------------------------------------------------------
# The replicated result over peer memory: gather and widening in ONE kernel per row block
# ---------------------------------------------------------------------------
_peer_ws = {}
_PEER_FLAG_WORDS = 64            # words 0..31: "row block i of call e is there"; word 32: "call e has been read"
_PEER_DONE = 32
_PEER_LIMIT_US = 2_000_000       # every flag wait in the kernels gives up after this long


def _peer_workspace(dev, M: int, n_loc: int, world: int, rank: int, group, elem_bytes: int = 2):
    """Symmetric memory of this rank (two send buffers, by call parity, and the flag words), mapped by
    every peer; None when the platform offers no peer mapping (the caller then takes the NCCL path)."""
    import ctypes as C
    import torch.distributed as dist
    key = (str(dev), M, n_loc, world, rank, id(group), elem_bytes)
    ws = _peer_ws.get(key)
    if ws is not None:
        return ws or None
    buf = hdl = None
    ptrs = []
    try:
        import torch.distributed._symmetric_memory as symm
        send_bytes = (M * n_loc * elem_bytes + 255) // 256 * 256
        total = 2 * send_bytes + 4 * _PEER_FLAG_WORDS
        buf = symm.empty(total, dtype=torch.uint8, device=dev)
        buf.zero_()
        hdl = symm.rendezvous(buf, group if group is not None else dist.group.WORLD)
        ptrs = [int(x) for x in hdl.buffer_ptrs]
        mine = len(ptrs) == world and all(ptrs)
    except Exception:
        mine = False
    # the choice of path must be the same on every rank (one rank on NCCL and the others on peer
    # memory would wait for each other), and every rank's flag words must be zero before anyone reads them
    torch.cuda.synchronize(dev)
    agreed = torch.tensor([1 if mine else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
    if int(agreed.item()) == 0:                      # no symmetric memory here: remember, and use NCCL
        _peer_ws[key] = False
        return None
    arr = C.c_void_p * world
    ws = {
        "buf": buf, "hdl": hdl, "epoch": 0, "send_bytes": send_bytes,
        "send": [arr(*[p + q * send_bytes for p in ptrs]) for q in (0, 1)],
        "flags": arr(*[p + 2 * send_bytes for p in ptrs]),
        "own_flags": ptrs[rank] + 2 * send_bytes,
        "c_all": None,                               # int32 blocks: only when the int16 GEMM does not take the shape
    }
    _peer_ws.clear()                                 # one shape at a time, like the NCCL scratch
    _peer_ws[key] = ws
    return ws


def _gather_peer_blocks(a_packed, b_local, K: int, world: int, rank: int, group, row_blocks: Optional[int],
                        leave_sms: Optional[int] = None, ctas_per_peer: Optional[int] = None):
    """``_gather_row_blocks`` without NCCL and without the staged copy: this rank narrows each row block
    of its C into memory its peers have mapped and raises a flag; one kernel per row block, on a second
    stream, waits for each peer's flag, reads that peer's int16 block over NVLink and writes the widened
    values into the replicated result (``brute_b200_gather_peer_widen``). Returns None when peer
    mapping is not available or the shard width is not a multiple of 8 (4 for K > 32767, where the blocks
    travel as int32)."""
    from . import _lib as L
    lib = L.load()
    M, n_loc = int(a_packed.shape[0]), int(b_local.shape[0])
    dev = a_packed.device
    eb = 2 if int(K) <= 32767 else 4         # int16 blocks where |C| <= K fits, else the int32 blocks as they are
    if dev.type != "cuda" or n_loc % (16 // eb) or world > 16 or M == 0 or n_loc == 0:
        return None
    ws = _peer_workspace(dev, M, n_loc, world, rank, group, eb)
    if ws is None:
        return None
    nb = int(row_blocks) if row_blocks else max(1, min(4, M // 2048))
    nb = max(1, min(nb, M, 32))
    # Measured at 16384^3 (sweeps over row blocks x SMs left x CTAs per peer): on 8 GPUs the call is fastest
    # with ONE gather CTA per SM that the GEMM leaves free (56 left, 7 CTAs per peer: 0.894 ms against
    # 1.32 ms for NCCL + widening pass); on 2 GPUs, where the GEMM of a row block is four times longer,
    # with 32 SMs left and 32 CTAs for the one peer (1.74 against 2.04 ms).
    if leave_sms is None:
        leave_sms = 32 if world == 2 else 56
    if not ctas_per_peer:
        ctas_per_peer = 32 if world == 2 else max(2, int(leave_sms) // world)
    bounds = [b for b in (shard_bounds(M, nb, i) for i in range(nb)) if b[1] > b[0]]
    ws["epoch"] += 1
    e = ws["epoch"]
    q = e & 1
    out = torch.empty((M, world * n_loc), dtype=torch.int32, device=dev)
    send_q = ws["buf"][q * ws["send_bytes"]:q * ws["send_bytes"] + M * n_loc * eb].view(torch.int16 if eb == 2 else torch.int32).view(M, n_loc)
    cur = torch.cuda.current_stream(dev)
    comm = _comm_stream(dev)
    comm.wait_stream(cur)
    fused_ok = (a_packed.is_contiguous() and b_local.is_contiguous() and a_packed.dtype == torch.int64
                and b_local.dtype == torch.int64 and os.environ.get("BRUTE_B200_GATHER_FUSED", "1") != "0")
    with torch.cuda.device(dev):
        if e > 2:   # the peers have read what this buffer held two calls ago
            L.check(lib.brute_b200_peer_wait_flags(ws["send"][q], ws["flags"], world, rank, _PEER_DONE, e - 2,
                                                   _PEER_LIMIT_US, cur.cuda_stream), "peer_wait_flags")
        for i, (m0, m1) in enumerate(bounds):
            leave = int(leave_sms) if i > 0 else 0
            # the GEMM writes its int16 block straight into the symmetric buffer where the pair kernel takes
            # the operands; otherwise int32 GEMM + narrowing pass
            a_blk = a_packed[m0:m1]
            rc = L.UNSUPPORTED
            if eb == 4:                              # K > 32767: the int32 GEMM writes into the exchange buffer itself
                _ops.xnor_popcount_matmul_out(a_blk, b_local, K, leave, send_q[m0:m1])
                rc = L.OK
            elif fused_ok:
                rc = lib.brute_b200_xnor_gemm_i16(a_blk.data_ptr(), b_local.data_ptr(), send_q[m0:m1].data_ptr(), m1 - m0, n_loc,
                                                  int(a_blk.shape[1]), int(K), n_loc, leave, cur.cuda_stream)
            if rc == L.UNSUPPORTED:
                fused_ok = False
                if ws["c_all"] is None:
                    ws["c_all"] = torch.empty((M, n_loc), dtype=torch.int32, device=dev)
                c = _ops.xnor_popcount_matmul_out(a_blk, b_local, K, leave, ws["c_all"][m0:m1])
                _ops.narrow_i32_i16_out(c, send_q[m0:m1])
            else:
                L.check(rc, "xnor_gemm_i16")
            L.check(lib.brute_b200_peer_set_flag(ws["own_flags"] + 4 * i, e, cur.cuda_stream), "peer_set_flag")
            ready = torch.cuda.Event()
            ready.record(cur)
            comm.wait_event(ready)                   # the own block is read without a flag
            L.check(lib.brute_b200_gather_peer_widen(ws["send"][q], ws["flags"], out.data_ptr(), M, n_loc, eb, m0, m1,
                                                     world, rank, i, e, int(ctas_per_peer), _PEER_LIMIT_US,
                                                     comm.cuda_stream), "gather_peer_widen")
        L.check(lib.brute_b200_peer_set_flag(ws["own_flags"] + 4 * _PEER_DONE, e, comm.cuda_stream), "peer_set_flag")
    done = torch.cuda.Event()
    done.record(comm)
    cur.wait_event(done)       # the caller's stream is behind every write to `out`: no record_stream needed
    return out


def peer_gather_status() -> int:
    """0, or 1 + the rank whose flag a bounded wait of the peer-gather kernels gave up on (synchronises)."""
    from . import _lib as L
    return int(L.load().brute_b200_peer_wait_status())


def release_gather_workspace() -> None:
    """Free the scratch that ``sharded_matmul(gather=True)`` keeps between calls of one shape."""
    _gather_ws.clear()
    _peer_ws.clear()


def sharded_matmul(a_packed: torch.Tensor, b_packed: torch.Tensor, K: int, group=None,
                   gather: bool = False, row_blocks: Optional[int] = None) -> torch.Tensor:
    """Column-sharded xnor GEMM: this rank computes C[:, lo:hi] for its block of
    B's rows. With ``gather`` the blocks are all-gathered (NCCL on GPUs) so that every rank
    returns the full [M, N] matrix; the collective is ordered behind the GEMM by events, with no
    host sync between (``_gather_row_blocks``)."""
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    N = b_packed.shape[0]
    lo, hi = shard_bounds(N, world, rank)
    if gather and world > 1 and N % world == 0:
        if a_packed.is_cuda and os.environ.get("BRUTE_B200_GATHER", "peer") == "peer":
            full = _gather_peer_blocks(a_packed, b_packed[lo:hi], K, world, rank, group, row_blocks)
            if full is not None:
                return full
        return _gather_row_blocks(a_packed, b_packed[lo:hi], K, world, group, row_blocks)
    c_local = _ops.xnor_popcount_matmul(a_packed, b_packed[lo:hi], K)
    if not gather or world == 1:
        return c_local
    M = a_packed.shape[0]
    # uneven blocks: pad every block to the widest one, gather, drop the padding
    widths = [shard_bounds(N, world, r)[1] - shard_bounds(N, world, r)[0] for r in range(world)]
    wmax = max(widths)
    padded = torch.zeros((M, wmax), dtype=c_local.dtype, device=c_local.device)
    padded[:, :hi - lo] = c_local
    stacked = torch.empty((world * M, wmax), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(stacked, padded, group=group)
    blocks = stacked.view(world, M, wmax)
    return torch.cat([blocks[r, :, :widths[r]] for r in range(world)], dim=1)


def sharded_attention(q: Tensor, k: Tensor, v: torch.Tensor, causal: bool = True,
                      scale: Optional[float] = None, group=None, gather: bool = False) -> torch.Tensor:
    """Binary attention sharded by batch x head: the B*H heads are independent, so this
    rank computes heads [lo, hi) of the flattened (batch, head) axis and no data crosses
    GPUs on the path. Returns bf16 [hi - lo, S, D]; with ``gather`` the blocks are
    all-gathered (NCCL on GPUs) and every rank returns the full [B, H, S, D]."""
    import torch.distributed as dist

    if not (_is_b1(q) and _is_b1(k)):
        raise TypeError("sharded_attention: q and k must be bit1 tensors")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    B, H, S, D = (int(x) for x in v.shape)
    if scale is None:
        scale = D ** -0.5
    lo, hi = shard_bounds(B * H, world, rank)
    qp = q._packed_buf_contig().reshape(1, B * H, S, -1)[:, lo:hi]
    kp = k._packed_buf_contig().reshape(1, B * H, S, -1)[:, lo:hi]
    vv = v.as_subclass(torch.Tensor).reshape(1, B * H, S, D)[:, lo:hi]
    if hi > lo:
        local = _ops.binary_attention(qp, kp, vv, bool(causal), float(scale))[0]
    else:
        local = torch.empty((0, S, D), dtype=v.dtype, device=v.device)
    if not gather:
        return local
    if world == 1:
        return local.reshape(B, H, S, D)
    counts = [shard_bounds(B * H, world, r)[1] - shard_bounds(B * H, world, r)[0] for r in range(world)]
    cmax = max(counts)
    if cmax == min(counts):
        full = torch.empty((B * H, S, D), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(full, local.contiguous(), group=group)
        return full.reshape(B, H, S, D)
    # uneven blocks: pad to the largest block, gather, drop the padding
    padded = torch.zeros((cmax, S, D), dtype=local.dtype, device=local.device)
    padded[:hi - lo] = local
    stacked = torch.empty((world * cmax, S, D), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(stacked, padded, group=group)
    blocks = stacked.view(world, cmax, S, D)
    return torch.cat([blocks[r, :counts[r]] for r in range(world)], dim=0).reshape(B, H, S, D)


_host_streams = {}


def host_matmul(a_host: torch.Tensor, b_host: torch.Tensor, K: int, out: Optional[torch.Tensor] = None,
                device=None, rows_per_block: int = 2048, impl: int = 0) -> torch.Tensor:
    """Packed A [M, Kp] and B [N, Kp] in host memory -> int32 C [M, N] in host memory (`out`,
    or a new pinned tensor). Pinned operands make every copy asynchronous.

    The int32 result is 32x the size of the packed operands, so its way back over PCIe is what
    an end-to-end call waits for. B goes to the device once; A goes up in blocks of
    `rows_per_block` rows, each block's GEMM runs as soon as its rows have landed, and its block
    of C leaves on a third stream while the next GEMM runs. Work is ordered after the caller's
    current stream and the current stream waits for the last copy, so CUDA events recorded
    around the call on the current stream bracket all of it. Call `torch.cuda.synchronize()` (or
    synchronise the current stream) before reading `out` on the host.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    M, Kp = a_host.shape
    N = b_host.shape[0]
    if b_host.shape[1] != Kp:
        raise RuntimeError("host_matmul: packed K mismatch")
    if out is None:
        out = torch.empty((M, N), dtype=torch.int32).pin_memory()
    if tuple(out.shape) != (M, N) or out.dtype != torch.int32 or out.is_cuda or not out.is_contiguous():
        raise RuntimeError("host_matmul: out must be a contiguous int32 [M, N] host tensor")
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    if key not in _host_streams:
        _host_streams[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    s_in, s_out = _host_streams[key]
    cur = torch.cuda.current_stream(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    with torch.cuda.stream(s_in):
        d_b = b_host.to(dev, non_blocking=True)
        d_b.record_stream(cur)
    step = max(1, int(rows_per_block))
    for lo in range(0, M, step):
        hi = min(M, lo + step)
        with torch.cuda.stream(s_in):
            d_a = a_host[lo:hi].to(dev, non_blocking=True)
            d_a.record_stream(cur)
            landed = torch.cuda.Event()
            landed.record(s_in)
        cur.wait_event(landed)
        c = _ops.xnor_popcount_matmul_impl(d_a, d_b, int(K), int(impl))
        done = torch.cuda.Event()
        done.record(cur)
        s_out.wait_event(done)
        with torch.cuda.stream(s_out):
            out[lo:hi].copy_(c, non_blocking=True)
        c.record_stream(s_out)
    cur.wait_stream(s_out)
    return out
